"""Two mixers side by side that read the same input: each output is RMS-normalised over the model width with a gain of
its own, and the result is a weighted sum of the two (half and half: their mean).

    y = w_l * rms(left(x)) * gain_l + w_r * rms(right(x)) * gain_r

Either mixer is any registered mixer (softmax attention under a window beside a recurrence, say) with its own tensors under
its own prefix, and keeps what it keeps: the layer's cache need is the pair of theirs, and the layer's view of the cache a
pair of views.  The two norms and the sum are one kernel in float32.
"""
from __future__ import annotations

from ..config.spec import PartSpec
from ..errors import ConfigError
from ..kernels import ops
from .base import Mixer, WeightSpec, make_part, register_mixer


class PairedMixer(Mixer):
    """params: ``left`` and ``right`` ({"kind", "params", "prefix"}: a mixer each, the prefix local to this part), ``eps``,
    optional ``weights`` (default (0.5, 0.5)) and ``tensors``: local names of the gains ``left_norm``, ``right_norm``."""

    NAMES = {"left_norm": "left.out", "right_norm": "right.out"}

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.eps = float(params["eps"])
        self.weights = tuple(float(w) for w in params.get("weights", (0.5, 0.5)))
        if len(self.weights) != 2:
            raise ConfigError("paired mixer: one weight per side")
        self.names = dict(self.NAMES, **(params.get("tensors") or {}))
        self.sides = []
        for side in ("left", "right"):
            d = params[side]
            self.sides.append((str(d.get("prefix", side + ".")),
                               make_part("mixer", PartSpec(d["kind"], d.get("params", {})), hidden_size, runtime)))
        self.graph_safe = all(getattr(m, "graph_safe", True) for _, m in self.sides)
        self.gains = None

    def weight_specs(self):
        specs = {}
        for prefix, mixer in self.sides:
            for local, spec in mixer.weight_specs().items():
                specs[prefix + local] = spec
        for key in ("left_norm", "right_norm"):
            specs[self.names[key]] = WeightSpec((self.hidden_size,), "precise", ("one_plus_uniform", 0.1))
        return specs

    def optional_names(self):
        return {prefix + local for prefix, mixer in self.sides for local in mixer.optional_names()}

    def bind(self, tensors):
        for prefix, mixer in self.sides:
            mixer.bind({local: tensors[prefix + local] for local in mixer.weight_specs()})
        self.gains = tuple(tensors[self.names[key]].contiguous() for key in ("left_norm", "right_norm"))

    def weight_bytes(self):
        return sum(m.weight_bytes() for _, m in self.sides)

    def cache_need(self):
        return tuple(m.cache_need() for _, m in self.sides)

    def forward(self, x, step, cache_view):
        x = ops.resolve(x)                         # a plain tensor: two mixers read it
        left, right = (ops.resolve(m.forward(x, step, view)) for (_, m), view in zip(self.sides, cache_view))
        return ops.pair_norm_sum(left, right, self.gains[0], self.gains[1], self.eps, self.weights[0], self.weights[1])


register_mixer("paired", PairedMixer)
