"""The gated delta rule with a decay per key channel: a recurrent mixer whose state is a matrix per head.

    q, k, v = silu(conv(Wq x)), silu(conv(Wk x)), silu(conv(Wv x))     (a short causal convolution per channel)
    q, k    = unit vectors per head (x / sqrt(sum x^2 + unit_eps)); q also times dim^-1/2
    beta    = sigmoid(Wb x)                                             (one step size per head)
    g       = exp(-exp(A_h) softplus(A2 (A1 x) + dt))                   (one decay per head and key channel)
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   (the read-out sees the token's own write)
    y = Wo concat_heads(rms(o) * gain * sigmoid(G2 (G1 x)))

Value heads share query/key heads in groups (head h reads q/k head h // (heads / kv_heads)).  The projections that read
x (q, k, v, the two low-rank first factors and the step size) are one stacked matrix, so one product feeds the rest; the
two second factors are one product each (the decay's leaves its result in float32).  What a sequence carries - every
head's state and the convolutions' last taps - 1 inputs - is the layer execution's fixed-size cache entry, one float32
vector per slot, zero when a sequence opens; convolution sums, unit lengths, step sizes, decays, the recurrence and the
per-head norm are float32 in either run dtype.  The kernels walk a sequence's new tokens in order from that entry, so
prompts, parts of prompts and decoded tokens are one code path.

Two simpler forms, each a parameter: ``decay`` "head" - one decay per head, g = exp(-exp(A_h) softplus(a_h . x + dt_h)),
from a projection of its own with one row per head (no low-rank pair), the same for all key channels of the head; and
``gate`` {"activation": "silu", "rank": None} - the read-out's gate comes from one full projection and passes through
silu instead of the sigmoid.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import ops
from .attention import BRANCH_DTYPE
from .base import CacheNeed, Mixer, WeightSpec, register_mixer


class ChannelDeltaMixer(Mixer):
    """params: ``n_heads``, ``n_kv_heads``, ``key_dim``, ``value_dim`` (per head), ``taps`` (of the convolutions), ``eps``
    (of the per-head norm), ``unit_eps`` (inside the root of the unit lengths); optional ``decay_rank`` and ``gate_rank``
    (the sizes the random-weights mode gives the two low-rank pairs; a checkpoint's own are read from its tensors) and
    ``tensors``: local names; ``decay`` ("channel", or "head": tensor ``decay_head`` [heads, H] and ``decay_bias`` [heads]
    instead of the low-rank pair); ``gate`` ({"activation": "sigmoid" | "silu", "rank": "low" | None}; with rank None the
    tensor ``gate_full`` [heads * value_dim, H] replaces the pair)."""

    NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b",
             "rate": "A_log", "norm": "norm", "decay_in": "a1", "decay_out": "a2", "decay_bias": "dt_bias",
             "gate_in": "g1", "gate_out": "g2", "out": "o", "decay_head": "a", "gate_full": "g"}
    ROW_STEP = 16                # the stacked matrix's rows are a multiple of this: its product's rows stay 16-byte aligned
    MAX_KEY_DIM, MAX_TAPS = 512, 64      # what the scan keeps in a lane's registers, and the convolution in a thread's

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.key_dim = int(params["key_dim"])
        self.value_dim = int(params["value_dim"])
        self.taps = int(params["taps"])
        self.eps = float(params["eps"])
        self.unit_eps = float(params["unit_eps"])
        self.decay_rank = int(params.get("decay_rank", 16))
        self.gate_rank = int(params.get("gate_rank", 16))
        self.head_decay = params.get("decay", "channel") == "head"
        if params.get("decay", "channel") not in ("channel", "head"):
            raise ConfigError("channel delta: a decay per 'channel' or per 'head'")
        gate = params.get("gate") or {}
        self.gate_activation = str(gate.get("activation", "sigmoid"))
        self.gate_low_rank = gate.get("rank", "low") is not None
        if self.gate_activation not in ops.HEAD_GATES:
            raise ConfigError(f"channel delta: unknown gate activation {self.gate_activation!r}; known: {sorted(ops.HEAD_GATES)}")
        if min(self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim, self.taps, self.decay_rank, self.gate_rank) <= 0:
            raise ConfigError("channel delta: heads, sizes and taps must be positive")
        if self.key_dim > self.MAX_KEY_DIM or self.taps > self.MAX_TAPS:
            raise ConfigError(f"channel delta: the kernels take up to {self.MAX_KEY_DIM} key channels a head and convolutions of up "
                              f"to {self.MAX_TAPS} taps, not {self.key_dim} and {self.taps}")
        if self.n_heads % self.n_kv_heads:
            raise ConfigError(f"channel delta: {self.n_heads} heads are not a multiple of {self.n_kv_heads} query/key heads")
        self.names = dict(self.NAMES, **(params.get("tensors") or {}))
        self.qk_width = self.n_kv_heads * self.key_dim
        self.v_width = self.n_heads * self.value_dim
        self.channels = 2 * self.qk_width + self.v_width
        self.state_size = self.n_heads * self.key_dim * self.value_dim
        self.w_in = self.w_decay = self.w_gate = self.conv = self.decay_bias = self.rate = self.norm_gain = self.w_o = None

    def weight_specs(self):
        h, n, H, d = self.hidden_size, self.names, self.n_heads, self.key_dim
        conv = ("normal", 0.5)
        return {n["q"]: WeightSpec((self.qk_width, h), init=("normal", 0.1)),
                n["q_conv"]: WeightSpec((self.qk_width, self.taps), init=conv),
                n["k"]: WeightSpec((self.qk_width, h), init=("normal", 0.1)),
                n["k_conv"]: WeightSpec((self.qk_width, self.taps), init=conv),
                n["v"]: WeightSpec((self.v_width, h), init=("normal", 0.1)),
                n["v_conv"]: WeightSpec((self.v_width, self.taps), init=conv),
                n["beta"]: WeightSpec((H, h), init=("normal", 0.1)),
                n["rate"]: WeightSpec((H,), "precise", ("normal", 0.5)),
                n["norm"]: WeightSpec((self.value_dim,), "precise", ("one_plus_uniform", 0.1)),
                **({n["decay_head"]: WeightSpec((H, h), init=("normal", 0.1)),
                    n["decay_bias"]: WeightSpec((H,), "precise", ("normal", 1.0))} if self.head_decay else
                   {n["decay_in"]: WeightSpec((self.decay_rank, h), free_dims=(0,)),
                    n["decay_out"]: WeightSpec((H * d, self.decay_rank), init=("normal", 0.2), free_dims=(1,)),
                    n["decay_bias"]: WeightSpec((H * d,), "precise", ("normal", 1.0))}),
                **({n["gate_in"]: WeightSpec((self.gate_rank, h), free_dims=(0,)),
                    n["gate_out"]: WeightSpec((self.v_width, self.gate_rank), init=("normal", 0.2), free_dims=(1,))}
                   if self.gate_low_rank else {n["gate_full"]: WeightSpec((self.v_width, h))}),
                n["out"]: WeightSpec((h, self.v_width))}

    def bind(self, tensors):
        n = self.names
        pairs = ([] if self.head_decay else [("decay_in", "decay_out", "decay")]) + \
            ([("gate_in", "gate_out", "gate")] if self.gate_low_rank else [])
        for a, b, what in pairs:
            if tensors[n[a]].shape[0] != tensors[n[b]].shape[1]:
                raise ConfigError(f"channel delta: the two factors of the {what} do not share a rank")
        # the stacked matrix's rows: q, k, v channels; what feeds the decay (the low-rank pair's first factor, or a row per
        # head); what feeds the gate (the pair's first factor, or the whole gate); the step sizes
        decay_rows = tensors[n["decay_in"]] if not self.head_decay else tensors[n["decay_head"]][:0]   # per head: a product of its own
        gate_rows = tensors[n["gate_in"]] if self.gate_low_rank else tensors[n["gate_full"]]
        self.decay_rank = int(decay_rows.shape[0])
        self.gate_rank = int(gate_rows.shape[0])
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], decay_rows, gate_rows, tensors[n["beta"]]]
        pad = -sum(r.shape[0] for r in rows) % self.ROW_STEP
        if pad:
            rows.append(torch.zeros((pad, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.conv = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]], dim=0).contiguous()
        if self.head_decay:                          # rows of zeros up to a multiple of eight: the library's product likes whole eights
            a = tensors[n["decay_head"]]
            self.w_decay = torch.cat([a, torch.zeros((-a.shape[0] % 8, a.shape[1]), dtype=a.dtype, device=a.device)], dim=0).contiguous()
        else:
            self.w_decay = tensors[n["decay_out"]].contiguous()
        self.w_gate = tensors[n["gate_out"]].contiguous() if self.gate_low_rank else None
        self.decay_bias = tensors[n["decay_bias"]].contiguous()
        self.rate = tensors[n["rate"]].contiguous()
        self.norm_gain = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["out"]].contiguous()

    def weight_bytes(self):
        mats = (self.w_in, self.conv, self.w_decay, self.w_gate, self.w_o)
        return sum(m.numel() for m in mats if m is not None) * self.w_in.element_size()

    def cache_need(self):
        # per slot: the heads' states, then the convolutions' last taps - 1 inputs
        return CacheNeed("state", state_shape=(self.state_size + (self.taps - 1) * self.channels,), state_dtype=torch.float32)

    def forward(self, x, step, cache_view):
        C, dr, gr = self.channels, self.decay_rank, self.gate_rank
        proj = ops.linear(x, self.w_in, resident=True)
        low_decay, low_gate, b = proj[:, C:C + dr], proj[:, C + dr:C + dr + gr], proj[:, C + dr + gr:C + dr + gr + self.n_heads]
        # decay logits leave their product in float32 (per head: a product of x with a row per head)
        z = ops.linear(x, self.w_decay, out_dtype=torch.float32, resident=True)[:, :self.n_heads] if self.head_decay else \
            ops.linear(low_decay, self.w_decay, out_dtype=torch.float32, resident=True)
        gate = ops.linear(low_gate, self.w_gate, resident=True) if self.gate_low_rank else low_gate
        o = ops.delta_rule(proj, self.conv, b, z, self.decay_bias, self.rate, step.token_seq, step.cu_new, cache_view.slots,
                           cache_view.state, self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim,
                           self.key_dim ** -0.5, self.unit_eps, head_decay=self.head_decay)
        y = ops.head_norm_gate(o, gate, self.norm_gain, self.n_heads, self.value_dim, self.eps, self.runtime.dtype,
                               gate=self.gate_activation)
        return ops.linear(y, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)


register_mixer("channel_delta", ChannelDeltaMixer)
