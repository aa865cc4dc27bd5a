"""RMSNorm over the float32 residual stream.

y = x / sqrt(mean(x^2) + eps) * gain, eps inside the root, no mean subtraction, gain used as
is (src/DotLLM.Cpu/Kernels/RmsNorm.cs:22-51).  The fused form adds a pending branch output
to the stream first, as the reference's fused_add_rmsnorm does
(native/kernels/fused_add_rmsnorm.cu:9-72).
"""
from __future__ import annotations

from ..errors import ConfigError
from ..kernels import ops
from .base import Norm, WeightSpec, register_norm


class RmsNorm(Norm):
    """params: ``eps``; optional ``gain_init`` for the random-weights mode; optional ``offset``: the stored
    tensor is the gain minus this number (1.0: a gain kept around zero, y = rms(x) * (1 + w); the sum is
    taken once, in float32, when the weights are bound); optional ``tensor``: the local name of the stored
    tensor (default "weight"; "" when the prefix is the whole name)."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.eps = float(params["eps"])
        self.offset = float(params.get("offset", 0.0))
        self.tensor_name = str(params.get("tensor", "weight"))
        self.gain = None

    def weight_specs(self):
        default = ("ones",) if self.offset == 0.0 else ("normal", 0.1)
        return {self.tensor_name: WeightSpec((self.hidden_size,), "precise",
                                             tuple(self.params.get("gain_init", default)))}

    def bind(self, tensors):
        stored = tensors[self.tensor_name]
        self.gain = stored if self.offset == 0.0 else (stored + self.offset).contiguous()

    def branch(self, data):
        return ops.NormedBranch(data, self.gain, self.eps)

    def weight_bytes(self):
        return self.gain.numel() * self.gain.element_size()

    fuses_products = True

    def forward(self, x):
        return ops.add_rmsnorm(x, None, self.gain, self.eps, self.runtime.dtype)

    def add_forward(self, residual, delta, lazy=False):
        return ops.add_rmsnorm(residual, delta, self.gain, self.eps, self.runtime.dtype, lazy=lazy)


class StreamNorm(Norm):
    """A norm that reads a residual stream kept as ``copies`` copies (one float32 row [copies * H] per token): it sees the
    weighted sum of the copies - every copy once where nobody gives weights, which is the model's result - after adding
    what the sublayer before left unadded (``ops.StreamWrite``), all in one kernel.

    params: ``eps``; ``kind`` "layernorm" ((u - mean) / sqrt(mean((u - mean)^2) + eps) * gain + bias) or "rmsnorm"
    (u / sqrt(mean(u^2) + eps) * gain, no bias); ``copies`` (default 1); optional ``tensor`` and ``bias_tensor``: the local
    names of gain and bias (default "weight", "bias")."""

    reads_streams = True

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.eps = float(params["eps"])
        self.kind = str(params.get("kind", "layernorm"))
        if self.kind not in ops.STREAM_NORMS:
            raise ConfigError(f"stream norm: unknown kind {self.kind!r}; known: {sorted(ops.STREAM_NORMS)}")
        self.copies = int(params.get("copies") or 1)
        self.gain_name = str(params.get("tensor", "weight"))
        self.bias_name = str(params.get("bias_tensor", "bias"))
        self.gain = self.bias = None

    def weight_specs(self):
        specs = {self.gain_name: WeightSpec((self.hidden_size,), "precise", ("one_plus_uniform", 0.1))}
        if self.kind == "layernorm":
            specs[self.bias_name] = WeightSpec((self.hidden_size,), "precise", ("normal", 0.1))
        return specs

    def bind(self, tensors):
        self.gain = tensors[self.gain_name].contiguous()
        self.bias = tensors[self.bias_name].contiguous() if self.kind == "layernorm" else None

    def weight_bytes(self):
        return self.gain.numel() * 4 * (2 if self.bias is not None else 1)

    def read_stream(self, stream, copies, pending, read_weights):
        if pending is not None and not isinstance(pending, ops.StreamWrite):
            raise ConfigError("stream norm: what joins a stream of copies must come from a stream connection")
        return ops.stream_norm(stream, copies, pending, read_weights, self.gain, self.bias, self.eps, self.runtime.dtype, kind=self.kind)

    def forward(self, x):
        return self.read_stream(x, self.copies, None, None)

    def add_forward(self, residual, delta):
        return self.read_stream(residual, self.copies, delta, None)


register_norm("rmsnorm", RmsNorm)
register_norm("stream_norm", StreamNorm)
