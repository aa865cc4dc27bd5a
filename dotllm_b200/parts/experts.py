"""A feed-forward of many small gated experts, a few per token, with an optional expert that every token uses.

    z = R x + b (float32);  chosen = the ``top`` largest z;  weights = softmax over the chosen z alone
    y = sum over chosen e of weight_e * D_e act(G_e x, U_e x)   (+ Ds act(Gs x, Us x), the shared expert)

Variants, each a parameter: an activation of one product instead of a gating (``activation`` in ``ops.UNGATED``, e.g.
"relu2": y = D_e relu(U_e x)^2, no gate matrices); ``scoring`` "sigmoid": the weights are the chosen experts' own
sigmoid(z), not renormalised; ``weight_on`` "input": the weight multiplies what goes into the expert, D_e act(U_e (w x)),
not what comes out; a shared expert with a gate of its own, sigmoid(g . x) per token (``shared.gate``: the gate's row
rides the router's product); a ``correction`` per expert that is added to the shares of the softmax over all experts for
the choice alone, chosen weights divided by their sum (``normalise``) and multiplied by a constant (``weight_scale``); and
``identity`` experts: the router's last that many outputs name experts without matrices whose output is their input.

Router, choice, the experts' products and the weighted sum are kernels that read the choice on the device,
so a step with this part can be captured in a graph.  The experts' matrices are stacked when the weights are
bound ([E, 2*ff, H] gate rows then up rows, and [E, H, ff]).
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..kernels import ops
from .base import FeedForward, WeightSpec, register_feed_forward


class RoutedExperts(FeedForward):
    """params: ``n_experts``, ``top``, ``intermediate_size`` (of one expert), ``activation`` (one of
    ``ops.GATINGS``) with ``limit`` and ``alpha``; ``router_bias`` (default True); ``shared``: None or
    {"intermediate_size", "limit", "gate"} (same activation and alpha; ``gate`` True: the shared expert's output is
    multiplied by sigmoid of a per-token logit, tensor ``shared_gate`` [1, H]); ``scoring`` ("softmax_chosen",
    "sigmoid", or "softmax_all": a chosen expert's share of the softmax over all experts, not renormalised),
    ``groups`` (None or (count, keep): the experts lie in ``count`` equal runs of neighbours, a run scores its best expert,
    and only the experts of the ``keep`` best runs can be chosen) and ``weight_on`` ("output" or "input"); optional ``tensors``: local name patterns ``expert`` (with
    {e} and {m} for the expert's index and gate / up / down), ``router``, ``router_bias``, ``shared`` (with {m}),
    ``shared_gate``, ``correction``.  With ``scoring`` "softmax_all": ``correction`` (True: tensor ``correction`` [experts +
    identity], added to the shares for the choice alone), ``normalise`` (the chosen weights are divided by their sum + 1e-20),
    ``weight_scale`` (they are multiplied by it) and ``identity`` (that many more router rows, for experts that give back
    their input times their weight; they have no matrices)."""

    ROUTER_ROW_STEP = 8
    NAMES = {"expert": "experts.{e}.{m}_proj.weight", "router": "router.weight", "router_bias": "router.bias",
             "shared": "shared_expert.{m}_proj.weight", "shared_gate": "shared_expert_gate.weight", "correction": "correction"}

    def __init__(self, params, hidden_size, runtime):
        super().__init__(params, hidden_size, runtime)
        self.n_experts = int(params["n_experts"])
        self.top = int(params["top"])
        self.ff = int(params["intermediate_size"])
        self.activation = params.get("activation", "silu")
        if self.activation not in ops.GATINGS:
            raise ConfigError(f"routed experts: unsupported activation {self.activation!r}; known: {sorted(ops.GATINGS)}")
        if not 0 < self.top <= self.n_experts + int(params.get("identity") or 0) or self.ff <= 0:
            raise ConfigError(f"routed experts: cannot use {self.top} of {self.n_experts} experts of width {self.ff}")
        self.limit = float(params.get("limit", 0.0))
        self.alpha = float(params.get("alpha", 1.0))
        self.router_bias = bool(params.get("router_bias", True))
        self.gated = self.activation not in ops.UNGATED
        self.scoring = params.get("scoring", "softmax_chosen")
        if self.scoring not in ops.ROUTER_SCORINGS:
            raise ConfigError(f"routed experts: unknown scoring {self.scoring!r}; known: {sorted(ops.ROUTER_SCORINGS)}")
        groups = params.get("groups")
        self.groups = (int(groups[0]), int(groups[1])) if groups else None
        if self.groups and (self.groups[0] <= 0 or self.n_experts % self.groups[0] or not 0 < self.groups[1] <= self.groups[0]
                            or self.top > self.groups[1] * (self.n_experts // self.groups[0])):
            raise ConfigError(f"routed experts: {self.n_experts} experts in {self.groups[0]} groups of which {self.groups[1]} "
                              f"stay cannot give {self.top} choices")
        self.identity = int(params.get("identity") or 0)
        self.correction = bool(params.get("correction", False))
        self.normalise = bool(params.get("normalise", False))
        self.weight_scale = float(params.get("weight_scale", 1.0))
        if (self.identity or self.correction or self.normalise or self.weight_scale != 1.0) and (self.scoring != "softmax_all" or self.groups):
            raise ConfigError("routed experts: identity experts, a correction, normalised and scaled weights go with the softmax over all "
                              "experts, without groups")
        if self.identity < 0 or self.top > self.n_experts + self.identity:
            raise ConfigError(f"routed experts: cannot use {self.top} of {self.n_experts} + {self.identity} experts")
        self.weight_on = params.get("weight_on", "output")
        if self.identity and self.weight_on != "output":
            raise ConfigError("routed experts: identity experts are weighed on their output")
        if self.weight_on not in ("output", "input"):
            raise ConfigError(f"routed experts: weight_on is 'output' or 'input', not {self.weight_on!r}")
        shared = params.get("shared")
        self.shared_gate = bool(shared.get("gate", False)) if shared else False
        self.shared_ff = int(shared["intermediate_size"]) if shared else 0
        self.shared_limit = float(shared.get("limit", self.limit)) if shared else 0.0
        self.names = dict(self.NAMES, **(params.get("tensors") or {}))
        self.w_router = self.b_router = self.w_gate_up = self.w_down = self.ws_gate_up = self.ws_down = None

    def _expert(self, e, m):
        return self.names["expert"].format(e=e, m=m)

    def weight_specs(self):
        h = self.hidden_size
        specs = {}
        for e in range(self.n_experts):
            if self.gated:
                specs[self._expert(e, "gate")] = WeightSpec((self.ff, h))
            specs[self._expert(e, "up")] = WeightSpec((self.ff, h))
            specs[self._expert(e, "down")] = WeightSpec((h, self.ff))
        # random routers are drawn wide, so that the chosen logits stand clear of the others (few near-ties)
        specs[self.names["router"]] = WeightSpec((self.n_experts + self.identity, h), init=("normal", 0.5))
        if self.correction:
            specs[self.names["correction"]] = WeightSpec((self.n_experts + self.identity,), "precise", ("normal", 0.02))
        if self.router_bias:
            specs[self.names["router_bias"]] = WeightSpec((self.n_experts + self.identity,), "precise", ("normal", 0.5))
        if self.shared_ff:
            for m, shape in (("gate", (self.shared_ff, h)), ("up", (self.shared_ff, h)), ("down", (h, self.shared_ff))):
                if m != "gate" or self.gated:
                    specs[self.names["shared"].format(m=m)] = WeightSpec(shape)
            if self.shared_gate:
                specs[self.names["shared_gate"]] = WeightSpec((1, h), init=("normal", 0.1))
        return specs

    def bind(self, tensors):
        E = range(self.n_experts)
        if self.gated:
            self.w_gate_up = torch.stack([torch.cat([tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")]], dim=0)
                                          for e in E]).contiguous()
        else:
            self.w_gate_up = torch.stack([tensors[self._expert(e, "up")] for e in E]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")] for e in E]).contiguous()
        self.w_router = tensors[self.names["router"]].contiguous()
        self.b_router = tensors[self.names["router_bias"]].contiguous() if self.router_bias else None
        self.choice_correction = tensors[self.names["correction"]].contiguous() if self.correction else None
        pad = -self.w_router.shape[0] % self.ROUTER_ROW_STEP
        if pad and (self.identity or self.correction) and not self.shared_gate:       # rows of zeros: the library's product likes whole eights
            self.w_router = torch.cat([self.w_router, torch.zeros((pad, self.hidden_size), dtype=self.w_router.dtype,
                                                                  device=self.w_router.device)], dim=0).contiguous()
        if self.shared_ff:
            name = self.names["shared"]
            if self.gated:
                self.ws_gate_up = torch.cat([tensors[name.format(m="gate")], tensors[name.format(m="up")]], dim=0).contiguous()
            else:
                self.ws_gate_up = tensors[name.format(m="up")].contiguous()
            self.ws_down = tensors[name.format(m="down")].contiguous()
            if self.shared_gate:                     # the gate's row behind the experts' rows: one product gives both
                rows = [self.w_router, tensors[self.names["shared_gate"]]]
                pad = -(self.w_router.shape[0] + 1) % self.ROUTER_ROW_STEP       # rows of zeros: the library's product likes whole eights
                if pad:
                    rows.append(torch.zeros((pad, self.hidden_size), dtype=self.w_router.dtype, device=self.w_router.device))
                self.w_router = torch.cat(rows, dim=0).contiguous()

    def weight_bytes(self):
        """Bytes a decode step of one token reads: the router, the chosen experts and the shared one."""
        size = self.w_down.element_size()
        mats = 3 if self.gated else 2
        chosen = mats * self.ff * self.hidden_size * self.top
        shared = mats * self.shared_ff * self.hidden_size
        return (self.w_router.numel() + chosen + shared) * size

    def forward(self, x):
        ids, weights, z = ops.route_topk(x, self.w_router, self.b_router, self.top, scoring=self.scoring,
                                         experts=self.n_experts + self.identity, with_logits=True, groups=self.groups,
                                         correction=self.choice_correction, normalise=self.normalise, weight_scale=self.weight_scale)
        # ids from n_experts on name identity experts: the kernels below skip them as experts and add weight * x instead
        identity = (x, self.identity) if self.identity else None
        shared = shared_gate = None
        if self.shared_ff:
            if self.gated:
                s = ops.gated_linear(x, self.ws_gate_up, resident=True, kind=self.activation, limit=self.shared_limit, alpha=self.alpha)
            else:
                s = ops.activated_linear(x, self.ws_gate_up, self.activation, resident=True)
            shared = ops.linear(s, self.ws_down, out_dtype=torch.float32, resident=True)
            if self.shared_gate:
                shared_gate = z[:, self.n_experts + self.identity:self.n_experts + self.identity + 1]   # the row behind the experts' rows
        # the weight on the expert's input scales the rows that go in; nothing is left to weigh on the way out
        scale, weights = (weights, None) if self.weight_on == "input" else (None, weights)
        if ops.experts_grouped_takes(x, ids, self.w_gate_up, self.w_down):
            # many rows: sorted by expert, both products as tensor-core tiles
            return ops.experts_grouped(x, ids, weights, self.w_gate_up, self.w_down, self.activation, self.limit, self.alpha,
                                       addend=shared, row_scale=scale, addend_gate=shared_gate, identity=identity)
        h = ops.expert_gate_up(x, ids, self.w_gate_up, self.activation, self.limit, self.alpha, row_scale=scale)
        return ops.expert_down(h, ids, weights, self.w_down, addend=shared, addend_gate=shared_gate, identity=identity)


register_feed_forward("routed_experts", RoutedExperts)
