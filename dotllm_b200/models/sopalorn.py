"""The Sopalorn decoder as a model description.

Token embedding times a constant; a residual stream kept as several copies that every sublayer reads and writes with
weights of its own (or one stream), every branch under a gain per channel; pre-norm layers with a layer norm (gain and
bias); per layer one of three mixers - softmax attention with a norm over the whole query and key projections, a rotation
of interleaved pairs with blended frequencies, one added to the softmax's denominator, maybe another layer's keys and
values; linear attention with a constant decay per head; or a windowed attention with learned sinks beside a gated delta
rule, each output normalised over the width, half the sum - and a dense feed-forward with a clamped gating, experts chosen
by corrected shares of a softmax over all (some of them identities), or none; a last layer norm over the sum of the
copies, a head of its own, logits times a constant.
Tensor names: ``embed``, ``l<i>.norm1`` (+ ``.b``), ``l<i>.norm2``, ``l<i>.ls1/2``, ``l<i>.hc1/2.in|out|mix``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm`` (+ ``.b``), ``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sopalorn import SopalornConfig
from ..config.spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

UNIT_EPS = 1e-6                 # inside the root that makes the delta rule's queries and keys unit vectors: fixed by the design
NO_LIMIT = 3.0e38               # a dense feed-forward without a `limit` key clamps nothing
GATE_ALPHA = 1.702              # the dense feed-forward's gate is g sigmoid(1.702 g): fixed by the design


def _norm(cfg, name, copies=None):
    return PartSpec("stream_norm", {"eps": cfg.eps, "kind": "layernorm", "copies": copies or 1, "tensor": "", "bias_tensor": ".b"}, name)


def _connection(cfg, prefix, which):
    return PartSpec("stream_copies", {"copies": cfg.streams, "scale": True,
                                      "tensors": {"scale": f"ls{which}", "in": f"hc{which}.in", "out": f"hc{which}.out",
                                                  "mix": f"hc{which}.mix"}}, prefix)


def _attention(cfg, m, windowed_side):
    """An attention layer's mixer, or (``windowed_side``) the attention beside the delta rule."""
    params = {"n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale,
              "window": m.window, "tensors": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                                              "sink": "sink"}}
    if windowed_side:
        params.update(sink=True, position=None)
        return params
    position = None
    if m.rot is not None and m.rot.dims:
        scaling = None
        if m.rot.scaling:
            factor, original, fast, slow = m.rot.scaling
            scaling = {"rope_type": "yarn", "factor": factor, "original_max_position_embeddings": original,
                       "fast_turns": fast, "slow_turns": slow}
        position = {"kind": "rotary", "params": {"rotary_dim": m.rot.dims, "theta": m.rot.base, "head_dim": m.dim,
                                                 "max_positions": cfg.positions(), "scaling": scaling}}
    params.update(sink="zero", position=position, pairing="interleaved", qk_norm={"eps": cfg.eps, "over": "projection"},
                  own_kv=m.kv_from is None)
    return params


def _mixer(cfg, layer, prefix):
    m = layer.mixer
    if layer.type == "attention":
        return PartSpec("attention", _attention(cfg, m, False), prefix)
    if layer.type == "lightning":
        return PartSpec("decayed_linear_attention", {"n_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
                                                     "decay": list(m.decay), "eps": cfg.eps}, prefix)
    r = m.right
    delta = {"n_heads": r.heads, "n_kv_heads": r.kv_heads, "key_dim": r.dim, "value_dim": r.vdim, "taps": r.conv, "eps": cfg.eps,
             "unit_eps": UNIT_EPS, "decay": "head", "gate": {"activation": "silu", "rank": None}}
    return PartSpec("paired", {"eps": cfg.eps, "weights": (0.5, 0.5),
                               "left": {"kind": "attention", "params": _attention(cfg, m.left, True), "prefix": "left."},
                               "right": {"kind": "channel_delta", "params": delta, "prefix": "right."},
                               "tensors": {"left_norm": "left.out", "right_norm": "right.out"}}, prefix)


def _feed_forward(mlp, prefix):
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"intermediate_size": mlp.ff, "activation": "clamped_sigmoid", "limit": mlp.limit or NO_LIMIT,
                                      "alpha": GATE_ALPHA, "tensors": ("gate", "up", "down")}, prefix)
    return PartSpec("routed_experts",
                    {"n_experts": mlp.experts, "identity": mlp.identity, "top": mlp.top, "intermediate_size": mlp.ff,
                     "activation": "silu", "router_bias": False, "scoring": "softmax_all", "correction": True, "normalise": True,
                     "weight_scale": mlp.scale, "shared": None,
                     "tensors": {"expert": "e{e}.{m}", "router": "router", "correction": "correction"}}, prefix)


def build_sopalorn_spec(cfg: SopalornConfig) -> ModelSpec:
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = [LayerPart("mixer_norm", "norm", _norm(cfg, p + "norm1")),
                 LayerPart("mixer", "mixer", _mixer(cfg, layer, p + "mix.")),
                 LayerPart("mixer_connection", "connection", _connection(cfg, p, 1))]
        if layer.mlp is not None:
            parts += [LayerPart("feed_forward_norm", "norm", _norm(cfg, p + "norm2")),
                      LayerPart("feed_forward", "feed_forward", _feed_forward(layer.mlp, p + "mlp.")),
                      LayerPart("feed_forward_connection", "connection", _connection(cfg, p, 2))]
        layers.append(LayerSpec("connected", tuple(parts)))
        schedule.append(ScheduleEntry(i, cache_of=layer.mixer.kv_from if layer.type == "attention" else None))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=cfg.positions(),
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "tensor": "embed", "init_std": 1.0,
                                               "scale": cfg.embedding_scale, "copies": cfg.streams or 1}, ""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=_norm(cfg, "final.norm", copies=cfg.streams),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "tensor": "", "scale": cfg.logit_scale}, "head"),
        stop_token_ids=tuple(cfg.eos_token_id),
        bos_token_id=cfg.bos_token_id)


register_architecture("Sopalorn", SopalornConfig, build_sopalorn_spec, model_types=("sopalorn",))
