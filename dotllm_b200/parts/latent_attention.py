"""Attention whose keys and values are expanded from one small latent per token, and only the latent is cached.

    cq = rms(Wdq x) * gq,   q_h = Wuq_h cq                      (queries through a latent of their own)
    c  = rms(Wdkv x) * gc                                        (the cached latent, width r)
    k_h = Wuk_h c,  v_h = Wuv_h c,   score = (q_h . k_h) * scale, softmax over the visible keys, out = Wo concat(o_h)

With ``q_rank`` None the queries come straight from one projection, q_h = Wq_h x (tensor ``q``), and the design has no query
latent.  No position enters the scores.  Since k_h and v_h are linear in c, the expansion moves to the query side:
q_h . (Wuk_h c) = (Wuk_h^T q_h) . c and sum_j p_j Wuv_h c_j = Wuv_h (sum_j p_j c_j).  What runs over the cache
is therefore attention of H query heads of width r against ONE shared key/value head, the latent itself:
the paged cache of the layer holds c (as keys and, transposed, as values) and the library's own
attention kernels (prefill on tcgen05, decode over pages, windows, page recycling) serve it unchanged.
The two per-head changes of basis are batched products around the attention.
"""
from __future__ import annotations

import math

import torch

from ..errors import ConfigError
from ..kernels import ops
from .attention import BRANCH_DTYPE
from .base import CacheNeed, Mixer, WeightSpec, register_mixer


class LatentAttentionMixer(Mixer):
    """params: ``n_heads``, ``key_dim``, ``value_dim`` (per head), ``q_rank`` (None: queries without a latent), ``kv_rank`` (the latents),
    ``eps`` (of the latents' norms), optional ``scale`` (default key_dim^-1/2), ``window`` (None: every
    earlier key; w: a query sees itself and the w - 1 tokens before it), ``tensors`` (local names)."""

    NAMES = {"q_down": "q_a_proj.weight", "q_norm": "q_a_norm.weight", "q_up": "q_b_proj.weight",
             "kv_down": "kv_a_proj.weight", "kv_norm": "kv_a_norm.weight", "k_up": "k_b_proj.weight",
             "v_up": "v_b_proj.weight", "out": "o_proj.weight", "q": "q_proj.weight"}

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.n_heads = int(params["n_heads"])
        self.key_dim = int(params["key_dim"])
        self.value_dim = int(params["value_dim"])
        self.q_rank = int(params["q_rank"]) if params.get("q_rank") is not None else None
        self.kv_rank = int(params["kv_rank"])
        self.eps = float(params["eps"])
        if min(self.n_heads, self.key_dim, self.value_dim, self.q_rank if self.q_rank is not None else 1, self.kv_rank) <= 0:
            raise ConfigError("latent attention: heads and sizes must be positive")
        scale = params.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.key_dim)
        window = params.get("window")
        self.window = int(window) if window else None
        if self.window is not None and self.window < 1:
            raise ConfigError("latent attention: a window holds at least the token itself")
        self.names = dict(self.NAMES, **(params.get("tensors") or {}))
        self.w_dq = self.w_dkv = self.q_gain = self.kv_gain = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = None

    def weight_specs(self):
        h, n, H = self.hidden_size, self.names, self.n_heads
        if self.q_rank is None:
            queries = {n["q"]: WeightSpec((H * self.key_dim, h))}
        else:
            queries = {n["q_down"]: WeightSpec((self.q_rank, h)),
                       n["q_norm"]: WeightSpec((self.q_rank,), "precise", ("one_plus_uniform", 0.1)),
                       n["q_up"]: WeightSpec((H * self.key_dim, self.q_rank), init=("normal", 0.1))}
        return {**queries,
                n["kv_down"]: WeightSpec((self.kv_rank, h)),
                n["kv_norm"]: WeightSpec((self.kv_rank,), "precise", ("one_plus_uniform", 0.1)),
                n["k_up"]: WeightSpec((H * self.key_dim, self.kv_rank), init=("normal", 0.1)),
                n["v_up"]: WeightSpec((H * self.value_dim, self.kv_rank), init=("normal", 0.1)),
                n["out"]: WeightSpec((h, H * self.value_dim))}

    def bind(self, tensors):
        n, H = self.names, self.n_heads
        if self.q_rank is None:
            self.w_uq = tensors[n["q"]].contiguous()
        else:
            self.w_dq = tensors[n["q_down"]].contiguous()
            self.q_gain = tensors[n["q_norm"]].contiguous()
            self.w_uq = tensors[n["q_up"]].contiguous()
        self.w_dkv = tensors[n["kv_down"]].contiguous()
        self.kv_gain = tensors[n["kv_norm"]].contiguous()
        # [H, r, d]: the transposed key expansion of every head, applied to its query
        self.w_uk_t = tensors[n["k_up"]].view(H, self.key_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["v_up"]].view(H, self.value_dim, self.kv_rank).contiguous()
        self.w_o = tensors[n["out"]].contiguous()

    def weight_bytes(self):
        mats = (self.w_dq, self.w_dkv, self.w_uq, self.w_uk_t, self.w_uv, self.w_o)
        return sum(m.numel() for m in mats if m is not None) * self.w_o.element_size()

    def cache_need(self):
        # one shared head whose keys and values are both the latent
        return CacheNeed("kv", n_kv_heads=1, head_dim=self.kv_rank, window=self.window)

    def forward(self, x, step, cache_view):
        dtype = self.runtime.dtype
        if self.q_rank is None:
            cq = x
        else:
            cq = ops.add_rmsnorm(ops.linear(x, self.w_dq, out_dtype=torch.float32, resident=True), None, self.q_gain,
                                 self.eps, dtype)
        q = ops.linear_per_head(ops.linear(cq, self.w_uq, resident=True), self.w_uk_t)            # [T, H*r]
        if cache_view.writes:
            c = ops.add_rmsnorm(ops.linear(x, self.w_dkv, out_dtype=torch.float32, resident=True), None, self.kv_gain,
                                self.eps, dtype)
        else:                                   # reads another execution's latents
            c = None
        a = ops.rope_cache_attention(q, c, c, None, None, 0, step.token_seq, step.token_pos, cache_view.block_table,
                                     cache_view.k, cache_view.v, self.n_heads, 1, self.kv_rank, self.scale,
                                     int(self.window or 0), plan=step.attention_plan)
        o = ops.linear_per_head(a, self.w_uv)                                                      # [T, H*dv]
        return ops.linear(o, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)


register_mixer("latent_attention", LatentAttentionMixer)
