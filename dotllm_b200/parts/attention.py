"""Causal self-attention mixer: MHA or GQA over the paged cache, optional window.

Order of operations as in the reference's block
(src/DotLLM.Models/Architectures/TransformerModel.cs:235-302): Q/K/V projections, position
encoding of Q and K, cache write, attention of the new queries over everything cached, output
projection.  scale = 1/sqrt(head_dim) and query head h reads KV head h // (n_heads/n_kv_heads)
(src/DotLLM.Cpu/Kernels/Attention.cs:47,76,106).  The three projections are stacked into one
matrix when the weights are bound, so one product yields q, k and v side by side.

Options beyond the reference's block, each a parameter: values of another width than the keys (``value_dim``),
biases on the three projections (added in float32 by the kernel that rotates and writes the cache), a gate per
(token, query head) from a projection of the mixer's input (``gate`` "head_sigmoid": the head's output times
sigmoid of its logit, before the output projection; the gate's rows ride the stacked product), and an execution
that reads another execution's keys and values (the schedule's ``cache_of``: such a layer has no key and value
projections, ``own_kv`` False); values that are the keys as projected, before any norm or rotation (``values`` "keys": no
value projection); an RMS norm of every query and key head before the rotation, with one gain for the queries and one for
the keys (``qk_norm``), or an RMS norm over the whole query projection and over the whole key projection, all heads at once,
with a gain per channel (``qk_norm`` with ``over`` "projection"); a window that keeps a sequence's first tokens visible
(``keep_first``); a learned number per head in the softmax's denominator, a sink without key or value (``sink``), or a sink
of score zero without a tensor (``sink`` "zero": one is added to the denominator); and a rotation that pairs channel 2i
with 2i + 1 (``pairing`` "interleaved").

Interleaved pairs on kernels that pair channel i with i + r/2.  Scores do not change when the channels of q and k are
permuted alike, so for a rotation of the first r channels in interleaved pairs the rows of the q and k projections (and
the gains of a norm over the whole projection, which does not care about the order either) are reordered once, when the
weights are bound: within each head the even channels of the first r come first, then the odd ones, then the rest.  The
cache holds the keys in that order; a layer that reads another's cache has the same rotation and orders its queries the
same way.

Keys and values of different widths on the tensor cores.  The tensor-core attention kernels take one width for keys
and values (32, 64, 96 or 128).  In a bfloat16 run a mixer with these options whose widths differ, or are equal and none of
those four, therefore lays every head out at the smallest such width W that holds both (where one does): the stacked matrix gets rows of zeros behind each head's own rows (a
head's q, k and v then come out of the product W wide, the added channels exactly zero), the biases zeros in the same
places, the cache is W wide on both sides, and the output projection gets columns of zeros where the added value
channels arrive.  Zero key channels add nothing to a score and zero value channels give zero outputs that meet zero
columns, so the result is the unpadded one; the rotation's pairs (i, i + rot/2) lie in a head's first channels and do
not move.  A float32 run, and widths beyond 128, keep the true widths and run the generic kernel.

A rotation of a part of the head on the kernels that rotate whole heads.  The fused kernels (the decode attention that
rotates the step's own token, the 16-byte rotation kernel) pair channel i with channel i + W/2.  A rotation of the first
r < W channels pairs i with i + r/2.  Scores do not change when the channels of q and k are permuted alike, so in that
layout the rows of the q and k projections (and their biases) are reordered once, when the weights are bound: the r/2 first
members of the pairs to the head's channels 0 .., their partners to W/2 .., the unrotated channels behind each.  The
rotary tables are widened to W/2 columns with cos 1 and sin 0 behind the r/2 real ones; a pair that meets those comes
out as it went in, exactly.  What the cache holds are the keys in that order; a layer that reads another's cache
orders its queries the same way (same widths and the same r).
"""
from __future__ import annotations

import math

import torch

from ..config.spec import PartSpec
from ..errors import ConfigError
from ..kernels import ops
from .base import CacheNeed, Mixer, WeightSpec, make_part, register_mixer

# Branch outputs are handed to the residual add in float32.
BRANCH_DTYPE = torch.float32


class AttentionMixer(Mixer):
    """params: ``n_heads``, ``n_kv_heads``, ``head_dim``, ``window`` (None = all keys),
    ``position`` ({"kind", "params"} of a position encoding), optional ``scale``, optional ``score``
    ({"softcap": c, "slopes": [one per head]}: scores are capped and biased by distance before the
    softmax, which sends the mixer to the generic attention kernel); optional ``value_dim`` (per head, default
    ``head_dim``), ``bias`` (True: q, k and v have biases), ``gate`` (None or "head_sigmoid"), ``own_kv`` (False: no key
    and value projections, the layer reads another's cache) and ``tensors``: the local names of ``q``, ``k``, ``v``,
    ``o``, ``gate`` and the bias suffix ``bias`` (appended to a projection's name); optional ``values`` ("own", or "keys":
    v is k as projected, there is no value projection and ``value_dim`` is ``head_dim``), ``qk_norm`` ({"eps"}: tensors
    ``q_norm``, ``k_norm`` [head_dim]), ``keep_first`` (with a window: that many first tokens of a sequence stay visible) and
    ``sink`` (True: tensor ``sink`` [n_heads], exp(sink_h) joins head h's softmax denominator; "zero": no tensor, every
    head's denominator gets exp(0) = 1 more); ``qk_norm`` may carry ``over`` "projection" (one RMS over all the query
    channels of a token and one over all its key channels, tensors ``q_norm`` [n_heads * head_dim], ``k_norm``
    [n_kv_heads * head_dim]); ``pairing`` ("half", or "interleaved": the rotation pairs channel 2i with 2i + 1)."""

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "gate": "g_proj.weight", "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sink": "sinks"}
    GATES = (None, "head_sigmoid")
    ROW_STEP = 16                # the stacked matrix's rows are a multiple of this: its product's rows stay 16-byte aligned

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.head_dim = int(params["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ConfigError(f"{self.n_heads} query heads are not a multiple of {self.n_kv_heads} KV heads")
        self.window = params.get("window")
        self.scale = float(params.get("scale", 1.0 / math.sqrt(self.head_dim)))
        pos = params.get("position") or {"kind": "none", "params": {}}
        self.position = make_part("position_encoding", PartSpec(pos["kind"], pos.get("params", {})),
                                  hidden_size, runtime)
        self.graph_safe = bool(getattr(self.position, "graph_safe", True))
        score = params.get("score") or {}
        slopes = score.get("slopes")
        if slopes is not None and len(slopes) != self.n_heads:
            raise ConfigError(f"score slopes: {len(slopes)} values for {self.n_heads} heads")
        self.score_hook = ops.ScoreHook(score.get("softcap", 0.0),
                                        None if slopes is None else torch.tensor(list(slopes), dtype=torch.float32,
                                                                                 device=runtime.device))
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        self.bias = bool(params.get("bias", False))
        self.gate = params.get("gate")
        if self.gate not in self.GATES:
            raise ConfigError(f"attention: unknown gate {self.gate!r}; known: {list(self.GATES)}")
        self.own_kv = bool(params.get("own_kv", True))
        self.values = params.get("values", "own")
        if self.values not in ("own", "keys"):
            raise ConfigError(f"attention: values are 'own' or 'keys', not {self.values!r}")
        if self.values == "keys" and (self.value_dim != self.head_dim or self.bias):
            raise ConfigError("attention: values that are the keys have the keys' width and no biases")
        qk_norm = params.get("qk_norm")
        self.qk_norm_eps = float(qk_norm["eps"]) if qk_norm else None
        self.qk_norm_over = str(qk_norm.get("over", "head")) if qk_norm else None
        if self.qk_norm_over not in (None, "head", "projection"):
            raise ConfigError(f"attention: a query/key norm runs over a 'head' or the 'projection', not {self.qk_norm_over!r}")
        self.sink = bool(params.get("sink", False))
        self.zero_sink = params.get("sink") == "zero"
        self.pairing = str(params.get("pairing", "half"))
        if self.pairing not in ("half", "interleaved"):
            raise ConfigError(f"attention: rotation pairs are 'half' or 'interleaved', not {self.pairing!r}")
        self.keep_first = int(params.get("keep_first") or 0)
        if self.keep_first < 0 or (self.keep_first and not self.window):
            raise ConfigError("attention: kept first tokens need a window (and cannot be negative)")
        self.q_gain = self.k_gain = self.sinks = None
        self.names = dict(self.NAMES, **(params.get("tensors") or {}))
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv_heads * self.head_dim
        self.v_width = self.n_kv_heads * self.value_dim
        self.o_dim = self.n_heads * self.value_dim
        # the reference's block as it is (one matrix of q, k and v rows, nothing added): its fused paths apply
        self.plain = not self.bias and self.gate is None and self.value_dim == self.head_dim and self.own_kv \
            and self.values == "own" and self.qk_norm_eps is None and not self.sink and not self.keep_first \
            and params.get("pairing", "half") == "half"
        # heads keep their own width and channel order where a norm runs over them or the keys double as values
        as_stored = self.values == "keys" or self.qk_norm_eps is not None or params.get("pairing") == "interleaved"
        self.w_qkv = None
        self.w_o = None
        self.biases = None
        # the width every head is laid out at (see the module's text); head_dim / value_dim stay the stored widths
        self.lay_k, self.lay_v = self.head_dim, self.value_dim
        if runtime.dtype == torch.bfloat16 and not self.plain and not as_stored and \
                (self.value_dim != self.head_dim or self.head_dim not in self.TENSOR_CORE_WIDTHS):
            fits = [w for w in self.TENSOR_CORE_WIDTHS if w >= max(self.head_dim, self.value_dim)]
            if fits and self.n_heads // self.n_kv_heads <= 16:
                self.lay_k = self.lay_v = fits[0]
        # a partial rotation spread over the whole head (see the module's text): fused_rotary() gives (cos, sin, r)
        fused = self.position.fused_rotary()
        rd = int(fused[2]) if fused is not None else 0
        self.spread = bool(runtime.dtype == torch.bfloat16 and not self.plain and not as_stored and self.lay_k == self.lay_v
                           and self.lay_k in self.TENSOR_CORE_WIDTHS and 0 < rd < self.lay_k)
        self.rotation = None if fused is None else (self._wide_tables(fused[0], fused[1], rd, self.lay_k) + (self.lay_k,)
                                                    if self.spread else fused)
        self.spread_order = self._spread_order(rd, self.lay_k) if self.spread else None
        if self.pairing == "interleaved" and rd:
            if self.spread:
                raise ConfigError("attention: interleaved pairs go with heads kept at their stored width")
            # new channel -> old channel of a head: pairs (2i, 2i + 1) become pairs (i, i + rd/2)
            self.spread_order = list(range(0, rd, 2)) + list(range(1, rd, 2)) + list(range(rd, self.lay_k))

    TENSOR_CORE_WIDTHS = (32, 64, 96, 128)      # kernels.attention_fast.DECODE_HEAD_DIMS

    _WIDE_TABLES: dict = {}

    @classmethod
    def _wide_tables(cls, cos, sin, rd, width):
        """The rotary tables with width/2 columns: the rd/2 real ones, then cos 1 and sin 0.  Layers with equal tables
        share one pair."""
        key = (cos.data_ptr() if cos.device.type != "meta" else id(cos), width, str(cos.device))
        if key not in cls._WIDE_TABLES:
            wide_cos = torch.ones((cos.shape[0], width // 2), dtype=cos.dtype, device=cos.device)
            wide_sin = torch.zeros((sin.shape[0], width // 2), dtype=sin.dtype, device=sin.device)
            wide_cos[:, :rd // 2] = cos
            wide_sin[:, :rd // 2] = sin
            cls._WIDE_TABLES[key] = (wide_cos.contiguous(), wide_sin.contiguous(), cos)     # cos kept: its address is the key
        return cls._WIDE_TABLES[key][:2]

    @staticmethod
    def _spread_order(rd, width):
        """new channel -> old channel of a head: pairs (i, i + rd/2) become pairs (i, i + width/2)."""
        half, rest = rd // 2, (width - rd) // 2
        return list(range(half)) + list(range(rd, rd + rest)) + list(range(half, rd)) + list(range(rd + rest, width))

    def _reorder(self, t, heads):
        """The rows (or entries) of ``t``, ``heads`` blocks of lay_k, in the spread order within each block."""
        if self.spread_order is None:
            return t
        order = torch.tensor(self.spread_order, dtype=torch.long, device=t.device)
        return t.reshape(heads, self.lay_k, *t.shape[1:])[:, order].reshape(t.shape)

    @staticmethod
    def _widen(t, heads, width, to, dim=0):
        """``t`` with ``heads`` blocks of ``width`` along ``dim``, each block followed by zeros up to ``to``."""
        if to == width:
            return t
        shape = list(t.shape)
        shape[dim:dim + 1] = [heads, width]
        pad = list(shape)
        pad[dim + 1] = to - width
        out = torch.cat([t.reshape(shape), torch.zeros(pad, dtype=t.dtype, device=t.device)], dim=dim + 1)
        shape[dim:dim + 2] = [heads * to]
        return out.reshape(shape)

    def weight_specs(self):
        h, n = self.hidden_size, self.names
        specs = {n["q"]: WeightSpec((self.q_dim, h))}
        if self.own_kv:
            specs[n["k"]] = WeightSpec((self.kv_dim, h))
            if self.values == "own":
                specs[n["v"]] = WeightSpec((self.v_width, h))
        if self.bias:
            specs[n["q_bias"]] = WeightSpec((self.q_dim,), "precise", ("normal", 0.1))
            if self.own_kv:
                specs[n["k_bias"]] = WeightSpec((self.kv_dim,), "precise", ("normal", 0.1))
                specs[n["v_bias"]] = WeightSpec((self.v_width,), "precise", ("normal", 0.1))
        if self.gate:
            specs[n["gate"]] = WeightSpec((self.n_heads, h), init=("normal", 0.1))
        if self.qk_norm_eps is not None:
            whole = self.qk_norm_over == "projection"
            specs[n["q_norm"]] = WeightSpec((self.q_dim if whole else self.head_dim,), "precise", ("one_plus_uniform", 0.1))
            if self.own_kv:
                specs[n["k_norm"]] = WeightSpec((self.kv_dim if whole else self.head_dim,), "precise", ("one_plus_uniform", 0.1))
        if self.sink and not self.zero_sink:
            specs[n["sink"]] = WeightSpec((self.n_heads,), "precise", ("normal", 1.0))
        specs[n["o"]] = WeightSpec((h, self.o_dim))
        return specs

    def bind(self, tensors):
        n = self.names
        H, G, hd, vd, lk, lv = self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim, self.lay_k, self.lay_v
        rows = [self._reorder(self._widen(tensors[n["q"]], H, hd, lk), H)]
        if self.own_kv:
            rows.append(self._reorder(self._widen(tensors[n["k"]], G, hd, lk), G))
            if self.values == "own":
                rows.append(self._widen(tensors[n["v"]], G, vd, lv))
        if self.gate:
            rows.append(tensors[n["gate"]])
        if not self.plain:
            total = sum(r.shape[0] for r in rows)
            pad = -total % self.ROW_STEP
            if pad:
                rows.append(torch.zeros((pad, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.w_qkv = torch.cat(rows, dim=0).contiguous()
        self.w_o = self._widen(tensors[n["o"]], H, vd, lv, dim=1).contiguous()
        if self.qk_norm_eps is not None and self.qk_norm_over == "projection":
            # one gain per channel of the projection: they follow their channels into the kernels' order
            self.q_gain = self._reorder(tensors[n["q_norm"]], H).contiguous()
            self.k_gain = self._reorder(tensors[n["k_norm"]], G).contiguous() if self.own_kv else None
            self.qk_gain = torch.cat([self.q_gain, self.k_gain]).contiguous() if self.own_kv else self.q_gain
        elif self.qk_norm_eps is not None:
            if self.spread_order is not None:
                raise ConfigError("attention: a gain shared by the heads does not follow reordered channels")
            self.q_gain = tensors[n["q_norm"]].contiguous()
            self.k_gain = tensors[n["k_norm"]].contiguous() if self.own_kv else None
        if self.zero_sink:
            self.sinks = torch.zeros((H,), dtype=torch.float32, device=self.w_qkv.device)
        elif self.sink:
            self.sinks = tensors[n["sink"]].contiguous()
        if self.bias:
            self.biases = (self._reorder(self._widen(tensors[n["q_bias"]], H, hd, lk), H).contiguous(),
                           self._reorder(self._widen(tensors[n["k_bias"]], G, hd, lk), G).contiguous() if self.own_kv else None,
                           self._widen(tensors[n["v_bias"]], G, vd, lv).contiguous() if self.own_kv else None)

    def weight_bytes(self):
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()

    def cache_need(self):
        return CacheNeed("kv", n_kv_heads=self.n_kv_heads, head_dim=self.lay_k, window=self.window,
                         v_dim=self.lay_v if self.lay_v != self.lay_k else None, keep_first=self.keep_first)

    takes_scaled_rows = True                    # x goes straight into the Q/K/V product

    def _forward_general(self, x, step, cache_view):
        """With biases, a gate, values of their own width or another layer's cache: one stacked product (q, then k and v
        where the layer has its own, then the gate's logits), one kernel that adds the biases, rotates and writes the
        cache, attention (gated in its last step, or by a kernel behind the tensor-core ones), the output projection."""
        if cache_view.writes != self.own_kv:
            raise ConfigError("attention: a layer without key and value projections must read another layer's cache "
                              "(and one with them keeps its own)")
        lk, lv = self.lay_k, self.lay_v
        qd, kvd, vw = self.n_heads * lk, self.n_kv_heads * lk, self.n_kv_heads * lv
        y = ops.linear(x, self.w_qkv, resident=True)
        q, at = y[:, :qd], qd
        k = v = None
        if self.own_kv and self.values == "keys":
            k, at = y[:, at:at + kvd], at + kvd
            v = k                                   # as projected: the norm below writes its result elsewhere
        elif self.own_kv:
            k, v, at = y[:, at:at + kvd], y[:, at + kvd:at + kvd + vw], at + kvd + vw
        g = y[:, at:at + self.n_heads] if self.gate else None
        if self.qk_norm_eps is not None and self.qk_norm_over == "projection":
            if self.own_kv:
                normed = ops.group_rmsnorm(y[:, :qd + kvd], self.qk_gain, qd, kvd, self.qk_norm_eps)
                q, k = normed[:, :qd], normed[:, qd:]
            else:
                q = ops.group_rmsnorm(q, self.qk_gain, qd, 0, self.qk_norm_eps)
        elif self.qk_norm_eps is not None:
            if self.own_kv:
                normed = ops.head_rmsnorm(y[:, :qd + kvd], self.q_gain, self.n_heads, lk, self.qk_norm_eps, self.k_gain, self.n_kv_heads)
                q, k = normed[:, :qd], normed[:, qd:]
            else:
                q = ops.head_rmsnorm(q, self.q_gain, self.n_heads, lk, self.qk_norm_eps)
        fused = self.rotation
        if fused is None:
            if self.biases is not None:
                raise ConfigError("attention: biases need a position encoding that rides the cache-write kernel")
            self.position.apply(q, k, step.token_pos)
            cos = sin = None
            rotary_dim = 0
        else:
            cos, sin, rotary_dim = fused
        a = ops.rope_cache_attention(q, k, v, cos, sin, rotary_dim, step.token_seq, step.token_pos,
                                     cache_view.block_table, cache_view.k, cache_view.v,
                                     self.n_heads, self.n_kv_heads, lk, self.scale,
                                     int(self.window or 0), plan=step.attention_plan,
                                     score_hook=self.score_hook if self.score_hook else None,
                                     value_dim=lv, biases=self.biases, gate=g, keep_first=self.keep_first, sinks=self.sinks)
        return ops.linear(a, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)

    def forward(self, x, step, cache_view):
        if not self.plain:
            return self._forward_general(x, step, cache_view)
        qd, kvd = self.q_dim, self.kv_dim
        fused = self.position.fused_rotary()
        if cache_view.writes and fused is not None and fused[2]:
            # a prompt step: rotation and cache write in the product's epilogue, then attention over the cache
            q = ops.qkv_rope_cache(x, self.w_qkv, fused[0], fused[1], fused[2], step.token_seq, step.token_pos,
                                   cache_view.block_table, cache_view.k, cache_view.v, self.n_heads, self.n_kv_heads,
                                   self.head_dim)
            if q is not None:
                a = ops.attention(q, cache_view.k, cache_view.v, step.token_seq, step.token_pos, cache_view.block_table,
                                  self.n_heads, self.n_kv_heads, self.head_dim, self.scale, int(self.window or 0),
                                  plan=step.attention_plan, score_hook=self.score_hook if self.score_hook else None)
                return ops.linear(a, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)
        if cache_view.writes:
            qkv = ops.linear(x, self.w_qkv, resident=True)
            q, k, v = qkv[:, :qd], qkv[:, qd:qd + kvd], qkv[:, qd + kvd:]
        else:                                   # reads another execution's cache: only queries
            q, k, v = ops.linear(x, self.w_qkv[:qd], resident=True), None, None
        if fused is None:
            self.position.apply(q, k, step.token_pos)
            cos = sin = None
            rotary_dim = 0
        else:
            cos, sin, rotary_dim = fused
        # rotation, cache write and attention: one kernel for a decode step, two otherwise
        a = ops.rope_cache_attention(q, k, v, cos, sin, rotary_dim, step.token_seq, step.token_pos,
                                     cache_view.block_table, cache_view.k, cache_view.v,
                                     self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                     int(self.window or 0), plan=step.attention_plan,
                                     score_hook=self.score_hook if self.score_hook else None)
        return ops.linear(a, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)


register_mixer("attention", AttentionMixer)
