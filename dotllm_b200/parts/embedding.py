"""Token embedding and the output head.

Embedding: h[t] = E[token[t]], no scale
(src/DotLLM.Models/Architectures/TransformerModel.cs:729-749).  Head: logits = n W^T in
float32 without bias or soft-cap (TransformerModel.cs:411-416); a tied head uses the embedding
table (src/DotLLM.Models/Architectures/TransformerWeights.cs:205-220).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, WeightSpec, register_embedding, register_head


class TokenEmbedding(Part):
    """params: ``vocab_size``; optional ``tensor`` (the table's local name, default "weight"), ``init_std``, ``scale``
    (h[t] = E[token[t]] * scale, the product taken in float32) and ``copies`` (S > 1: the stream starts as S copies of that
    row side by side, float32 [T, S * H], for layers that keep a stream of copies)."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.tensor_name = str(params.get("tensor", "weight"))
        self.scale = float(params.get("scale", 1.0))
        self.copies = int(params.get("copies") or 1)
        self.table = None

    def weight_specs(self):
        return {self.tensor_name: WeightSpec((self.vocab_size, self.hidden_size),
                                             init=("normal", float(self.params.get("init_std", 0.02))))}

    def bind(self, tensors):
        self.table = tensors[self.tensor_name].contiguous()

    def forward(self, step):
        """The step's tokens (``step.tokens`` int32 [T]) -> float32 [T, H]: the start of the residual
        stream.  An embedding gets the whole StepContext: one that also encodes positions reads
        ``step.token_pos``."""
        if self.copies == 1 and self.scale == 1.0:
            return ops.gather_rows(self.table, step.tokens)
        return ops.embed_copies(self.table, step.tokens, self.copies, self.scale)


class TokenPositionEmbedding(Part):
    """Token embedding plus a learned vector per absolute position, neither scaled: h[t] = E[token] + P[pos].
    params: ``vocab_size``, ``max_positions``; optional ``token_tensor`` / ``position_tensor`` (local names,
    default "weight" and "positions.weight") and ``init_std`` (of both tables in the random-weights mode)."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.max_positions = int(params["max_positions"])
        self.token_name = str(params.get("token_tensor", "weight"))
        self.position_name = str(params.get("position_tensor", "positions.weight"))
        self.table = self.positions = None

    def weight_specs(self):
        init = ("normal", float(self.params.get("init_std", 0.02)))
        return {self.token_name: WeightSpec((self.vocab_size, self.hidden_size), init=init),
                self.position_name: WeightSpec((self.max_positions, self.hidden_size), init=init)}

    def bind(self, tensors):
        self.table = tensors[self.token_name].contiguous()
        self.positions = tensors[self.position_name].contiguous()

    def forward(self, step):
        return ops.embed_positions(self.table, self.positions, step.tokens, step.token_pos)


class LinearHead(Part):
    """params: ``vocab_size``; optional ``softcap`` (c > 0: logits become c tanh(logits / c)), ``scale`` (the logits are
    multiplied by it, in float32, before any cap) and ``tensor`` (the
    local name of the matrix, default "weight"; "" when the prefix is the whole name).  Whether its matrix is the
    embedding table is the model description's business (``ModelSpec.shared_weights``): the part is handed a
    [vocab, hidden] matrix either way."""

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.softcap = float(params.get("softcap") or 0.0)
        self.scale = float(params.get("scale", 1.0))
        self.tensor_name = str(params.get("tensor", "weight"))
        self.weight = None

    def weight_specs(self):
        return {self.tensor_name: WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors):
        w = tensors[self.tensor_name]
        self.weight = w if w.is_contiguous() else w.contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    takes_scaled_rows = True                    # x goes straight into the product

    def forward(self, x):
        """[R, H] in the run dtype -> float32 logits [R, vocab]."""
        logits = ops.linear(x, self.weight, out_dtype=torch.float32, resident=True)
        if self.scale != 1.0:
            logits = ops.scale_values(logits, self.scale)
        return ops.softcap(logits, self.softcap) if self.softcap > 0 else logits


register_embedding("token_embedding", TokenEmbedding)
register_embedding("token_position_embedding", TokenPositionEmbedding)
register_head("linear_head", LinearHead)
