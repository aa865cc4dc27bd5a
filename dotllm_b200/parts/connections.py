"""A residual stream kept as several copies that every sublayer reads and writes with weights of its own.

Instead of one stream x a token carries S copies x_1 .. x_S, all equal to the embedding output at the start.  A sublayer
with the vectors ``in`` [S], ``out`` [S] and the matrix ``mix`` [S, S] (indexed from, to) sees

    u = sum_s in[s] x_s,    y = sublayer(norm(u)),    x_t <- sum_s mix[s, t] x_s + out[t] * (scale .* y)

(every copy at once, from the old copies), and the model's result is the sum of the copies.  ``scale`` is a gain per
channel on the sublayer's output (a layer scale).  With one copy and no weights (``copies`` None) this is the ordinary
residual sum, x <- x + scale .* y, through the same kernel.

The stream is one float32 row [S * H] per token.  A sublayer's output is handed on unadded (``ops.StreamWrite``); the next
``read`` - the next sublayer's, across the layer boundary too, or the model's last norm - does the write, the read and the
norm in one pass over the row (``ops.stream_norm``).  All of it is float32.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import ops
from .base import Connection, WeightSpec, register_connection


class StreamConnection(Connection):
    """params: ``copies`` (S, or None: one stream and the plain residual sum, no weights but the scale), ``scale`` (True:
    a gain per channel on the sublayer's output); optional ``tensors``: local names of ``in``, ``out``, ``mix``, ``scale``."""

    NAMES = {"in": "in", "out": "out", "mix": "mix", "scale": "scale"}
    MAX_COPIES = 16               # ST_MAX_COPIES in csrc/streams.cu

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        copies = params.get("copies")
        self.weighted = copies is not None
        self.copies = int(copies) if self.weighted else 1
        if not 0 < self.copies <= self.MAX_COPIES:
            raise ConfigError(f"stream connection: {self.copies} copies; the kernel takes 1 to {self.MAX_COPIES}")
        self.scaled = bool(params.get("scale", False))
        self.names = dict(self.NAMES, **(params.get("tensors") or {}))
        self.scale = self.mix = self.out = self.read_weights = None

    def weight_specs(self):
        n, S = self.names, self.copies
        specs = {}
        if self.scaled:
            specs[n["scale"]] = WeightSpec((self.hidden_size,), "precise", ("uniform", 0.5, 1.5))
        if self.weighted:
            specs[n["in"]] = WeightSpec((S,), "precise", ("uniform", 0.5 / S, 1.5 / S))
            specs[n["out"]] = WeightSpec((S,), "precise", ("uniform", 0.5, 1.5))
            specs[n["mix"]] = WeightSpec((S, S), "precise", ("eye_plus_normal", 0.1))
        return specs

    def bind(self, tensors):
        n = self.names
        self.scale = tensors[n["scale"]].contiguous() if self.scaled else None
        if self.weighted:
            self.read_weights = tensors[n["in"]].contiguous()
            self.out = tensors[n["out"]].contiguous()
            self.mix = tensors[n["mix"]].contiguous()
        else:
            ones = torch.ones((1,), dtype=torch.float32, device=self.runtime.device)
            self.read_weights, self.out, self.mix = ones, ones, ones.reshape(1, 1)

    def read(self, norm, stream, pending):
        if not getattr(norm, "reads_streams", False):
            raise ConfigError(f"stream connection: the norm {type(norm).__name__} cannot read a stream of copies")
        return norm.read_stream(stream, self.copies, pending, self.read_weights)

    def write(self, data):
        return ops.StreamWrite(data, self.scale, self.mix, self.out)


register_connection("stream_copies", StreamConnection)
