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
    ``tensors``: local names."""

    NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b",
             "rate": "A_log", "norm": "norm", "decay_in": "a1", "decay_out": "a2", "decay_bias": "dt_bias",
             "gate_in": "g1", "gate_out": "g2", "out": "o"}
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
                n["decay_in"]: WeightSpec((self.decay_rank, h), free_dims=(0,)),
                n["decay_out"]: WeightSpec((H * d, self.decay_rank), init=("normal", 0.2), free_dims=(1,)),
                n["decay_bias"]: WeightSpec((H * d,), "precise", ("normal", 1.0)),
                n["gate_in"]: WeightSpec((self.gate_rank, h), free_dims=(0,)),
                n["gate_out"]: WeightSpec((self.v_width, self.gate_rank), init=("normal", 0.2), free_dims=(1,)),
                n["out"]: WeightSpec((h, self.v_width))}

    def bind(self, tensors):
        n = self.names
        for a, b, what in (("decay_in", "decay_out", "decay"), ("gate_in", "gate_out", "gate")):
            if tensors[n[a]].shape[0] != tensors[n[b]].shape[1]:
                raise ConfigError(f"channel delta: the two factors of the {what} do not share a rank")
        self.decay_rank = int(tensors[n["decay_in"]].shape[0])
        self.gate_rank = int(tensors[n["gate_in"]].shape[0])
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["decay_in"]], tensors[n["gate_in"]], tensors[n["beta"]]]
        pad = -sum(r.shape[0] for r in rows) % self.ROW_STEP
        if pad:
            rows.append(torch.zeros((pad, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.conv = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]], dim=0).contiguous()
        self.w_decay = tensors[n["decay_out"]].contiguous()
        self.w_gate = tensors[n["gate_out"]].contiguous()
        self.decay_bias = tensors[n["decay_bias"]].contiguous()
        self.rate = tensors[n["rate"]].contiguous()
        self.norm_gain = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["out"]].contiguous()

    def weight_bytes(self):
        mats = (self.w_in, self.conv, self.w_decay, self.w_gate, self.w_o)
        return sum(m.numel() for m in mats) * self.w_in.element_size()

    def cache_need(self):
        # per slot: the heads' states, then the convolutions' last taps - 1 inputs
        return CacheNeed("state", state_shape=(self.state_size + (self.taps - 1) * self.channels,), state_dtype=torch.float32)

    def forward(self, x, step, cache_view):
        C, dr, gr = self.channels, self.decay_rank, self.gate_rank
        proj = ops.linear(x, self.w_in, resident=True)
        low_decay, low_gate, b = proj[:, C:C + dr], proj[:, C + dr:C + dr + gr], proj[:, C + dr + gr:C + dr + gr + self.n_heads]
        z = ops.linear(low_decay, self.w_decay, out_dtype=torch.float32, resident=True)
        gate = ops.linear(low_gate, self.w_gate, resident=True)
        o = ops.delta_rule(proj, self.conv, b, z, self.decay_bias, self.rate, step.token_seq, step.cu_new, cache_view.slots,
                           cache_view.state, self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim,
                           self.key_dim ** -0.5, self.unit_eps)
        y = ops.head_norm_gate(o, gate, self.norm_gain, self.n_heads, self.value_dim, self.eps, self.runtime.dtype, gate="sigmoid")
        return ops.linear(y, self.w_o, out_dtype=BRANCH_DTYPE, resident=True, lazy=True)


register_mixer("channel_delta", ChannelDeltaMixer)
