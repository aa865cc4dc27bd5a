"""Gated linear attention: a recurrent mixer whose state is a matrix per head that decays per key channel.

    q = Wq x / sqrt(dim),  k = Wk x,  v = Wv x,  alpha = sigmoid(A2 (A1 x) + b)^(1/tau)
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
    y   = Wo (concat_heads(rms(o_t) * gain) * silu(Wg x))

The five projections that read x (q, k, v, the output gate and the low-rank decay's first factor) are one
stacked matrix, so one product feeds the scan.  The state is the layer execution's fixed-size cache entry
(float32, zero when a sequence opens, carried from step to step); the decay logits leave their product in
float32, and decays, recurrence and the per-head norm are float32 in either run dtype.  The scan walks a
sequence's new tokens in order from the cached state, so prompts, parts of prompts and decoded tokens
are one code path.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import ops
from .attention import BRANCH_DTYPE
from .base import CacheNeed, Mixer, WeightSpec, register_mixer


class GatedLinearAttentionMixer(Mixer):
    """params: ``n_heads``, ``key_dim``, ``value_dim`` (per head), ``tau`` (the decay's root), ``eps`` (of the
    per-head norm); optional ``decay_rank`` (the size the random-weights mode gives the low-rank decay; a
    checkpoint's own is read from its tensors) and ``tensors``: local names of q, k, v, gate, out, norm,
    decay_in, decay_out, decay_bias."""

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight",
             "out": "o_proj.weight", "norm": "norm.weight", "decay_in": "decay_in.weight",
             "decay_out": "decay_out.weight", "decay_bias": "decay_out.bias"}

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.n_heads = int(params["n_heads"])
        self.key_dim = int(params["key_dim"])
        self.value_dim = int(params["value_dim"])
        self.tau = float(params["tau"])
        self.eps = float(params["eps"])
        self.decay_rank = int(params.get("decay_rank", 16))
        if min(self.n_heads, self.key_dim, self.value_dim, self.decay_rank) <= 0 or self.tau <= 0:
            raise ConfigError("gated linear attention: heads, sizes and tau must be positive")
        self.names = dict(self.NAMES, **(params.get("tensors") or {}))
        self.k_width = self.n_heads * self.key_dim
        self.v_width = self.n_heads * self.value_dim
        self.w_in = self.w_decay = self.decay_bias = self.norm_gain = self.w_o = None

    def weight_specs(self):
        h, n = self.hidden_size, self.names
        return {n["q"]: WeightSpec((self.k_width, h)),
                n["k"]: WeightSpec((self.k_width, h)),
                n["v"]: WeightSpec((self.v_width, h)),
                n["gate"]: WeightSpec((self.v_width, h)),
                n["out"]: WeightSpec((h, self.v_width)),
                n["norm"]: WeightSpec((self.value_dim,), "precise", ("one_plus_uniform", 0.1)),
                n["decay_in"]: WeightSpec((self.decay_rank, h), free_dims=(0,)),
                n["decay_out"]: WeightSpec((self.k_width, self.decay_rank), init=("normal", 0.2), free_dims=(1,)),
                n["decay_bias"]: WeightSpec((self.k_width,), "precise", ("normal", 1.0))}

    def bind(self, tensors):
        n = self.names
        if tensors[n["decay_in"]].shape[0] != tensors[n["decay_out"]].shape[1]:
            raise ConfigError("gated linear attention: the two factors of the decay do not share a rank")
        self.decay_rank = int(tensors[n["decay_in"]].shape[0])
        self.w_in = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]],
                               tensors[n["decay_in"]]], dim=0).contiguous()
        self.w_decay = tensors[n["decay_out"]].contiguous()
        self.decay_bias = tensors[n["decay_bias"]].contiguous()
        self.norm_gain = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["out"]].contiguous()

    def weight_bytes(self):
        return (self.w_in.numel() + self.w_decay.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.n_heads, self.key_dim, self.value_dim), state_dtype=torch.float32)

    def forward(self, x, step, cache_view):
        kw, vw = self.k_width, self.v_width
        proj = ops.linear(x, self.w_in, resident=True)
        q, k, v = proj[:, :kw], proj[:, kw:2 * kw], proj[:, 2 * kw:2 * kw + vw]
        gate, low = proj[:, 2 * kw + vw:2 * kw + 2 * vw], proj[:, 2 * kw + 2 * vw:]
        z = ops.linear(low, self.w_decay, out_dtype=torch.float32, resident=True)
        o = ops.gla_scan(q, k, v, z, self.decay_bias, step.cu_new, cache_view.slots, cache_view.state,
                         self.n_heads, self.key_dim, self.value_dim, self.key_dim ** -0.5, self.tau)
        y = ops.head_norm_gate(o, gate, self.norm_gain, self.n_heads, self.value_dim, self.eps, self.runtime.dtype)
        return ops.linear(y, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)


class DecayedLinearAttentionMixer(Mixer):
    """Linear attention whose state decays by one constant per head (lightning attention):

        q, k, v = silu(Wq x), silu(Wk x), silu(Wv x)          (heads x dim, heads x dim, heads x vdim)
        S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t    (no other scale)
        y   = Wo (rms(concat_heads(o_t)) * gain * sigmoid(Wg x))   (one RMS over all heads' outputs together)

    The four projections that read x are one stacked matrix; the scan is the gated linear attention's kernel in its
    constant-decay form (silu inside, float32 state per slot, a sequence's new tokens walked in order from the cached
    state); the norm over the concatenated heads is the per-head norm kernel with one head as wide as all.

    params: ``n_heads``, ``key_dim``, ``value_dim`` (per head), ``decay`` (one number in (0, 1] per head), ``eps``; optional
    ``tensors``: local names of q, k, v, gate, out, norm."""

    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm"}
    ROW_STEP = 16

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.n_heads = int(params["n_heads"])
        self.key_dim = int(params["key_dim"])
        self.value_dim = int(params["value_dim"])
        self.eps = float(params["eps"])
        decay = [float(d) for d in params["decay"]]
        if min(self.n_heads, self.key_dim, self.value_dim) <= 0 or len(decay) != self.n_heads or not all(0.0 <= d <= 1.0 for d in decay):
            raise ConfigError("decayed linear attention: positive sizes and one decay in [0, 1] per head")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.names = dict(self.NAMES, **(params.get("tensors") or {}))
        self.k_width = self.n_heads * self.key_dim
        self.v_width = self.n_heads * self.value_dim
        self.w_in = self.norm_gain = self.w_o = None

    def weight_specs(self):
        h, n = self.hidden_size, self.names
        return {n["q"]: WeightSpec((self.k_width, h)),
                n["k"]: WeightSpec((self.k_width, h)),
                n["v"]: WeightSpec((self.v_width, h)),
                n["gate"]: WeightSpec((self.v_width, h)),
                n["out"]: WeightSpec((h, self.v_width)),
                n["norm"]: WeightSpec((self.v_width,), "precise", ("one_plus_uniform", 0.1))}

    def bind(self, tensors):
        n = self.names
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]]]
        pad = -sum(r.shape[0] for r in rows) % self.ROW_STEP
        if pad:
            rows.append(torch.zeros((pad, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.norm_gain = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["out"]].contiguous()

    def weight_bytes(self):
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.n_heads, self.key_dim, self.value_dim), state_dtype=torch.float32)

    def forward(self, x, step, cache_view):
        kw, vw = self.k_width, self.v_width
        proj = ops.linear(x, self.w_in, resident=True)
        q, k, v, gate = proj[:, :kw], proj[:, kw:2 * kw], proj[:, 2 * kw:2 * kw + vw], proj[:, 2 * kw + vw:2 * kw + 2 * vw]
        o = ops.gla_scan(q, k, v, None, self.decay, step.cu_new, cache_view.slots, cache_view.state, self.n_heads, self.key_dim,
                         self.value_dim, 1.0)
        y = ops.head_norm_gate(o, gate, self.norm_gain, 1, vw, self.eps, self.runtime.dtype, gate="sigmoid")
        return ops.linear(y, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)


register_mixer("gated_linear_attention", GatedLinearAttentionMixer)
register_mixer("decayed_linear_attention", DecayedLinearAttentionMixer)
