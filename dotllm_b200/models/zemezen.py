"""The Zemezen decoder as a model description.

Token embedding; layers that read the stream once, x += mixer(n(x)) + ff(n(x)) with one norm for both sublayers;
per layer one of three mixers - a gated delta rule whose state decays per key channel behind short convolutions
(a fixed-size state per sequence), attention over one cached latent per token, or attention whose values are its
unnormed, unrotated keys under a sliding window that also keeps the sequence's first tokens, with a learned sink in
the softmax's denominator - and a dense SwiGLU feed-forward, routed experts chosen among the best groups by a softmax
over all experts, or none; a layer may run with another layer's weights on a cache of its own; a final norm and a
head of its own.
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.zemezen import ZemezenConfig

UNIT_EPS = 1e-6                 # inside the root that makes the delta rule's queries and keys unit vectors: fixed by the design


def _norm(cfg, name):
    return PartSpec("rmsnorm", {"eps": cfg.eps, "tensor": ""}, name)


def _mixer(cfg, layer, prefix):
    m = layer.mixer
    if layer.type == "channel_delta":
        params = {"n_heads": m.heads, "n_kv_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim, "taps": m.conv,
                  "eps": cfg.eps, "unit_eps": UNIT_EPS}
        if m.ranks is not None:
            params["decay_rank"], params["gate_rank"] = m.ranks
        return PartSpec("channel_delta", params, prefix)
    if layer.type == "latent_attention":
        return PartSpec("latent_attention",
                        {"n_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "q_rank": None, "kv_rank": m.kv_rank,
                         "eps": cfg.eps, "scale": m.scale, "window": None,
                         "tensors": {"q": "q", "kv_down": "dkv", "kv_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "out": "o"}},
                        prefix)
    position = None
    if m.rot_dims:
        position = {"kind": "rotary", "params": {"rotary_dim": m.rot_dims, "theta": m.rot_base, "head_dim": m.dim,
                                                 "max_positions": cfg.positions(), "scaling": None}}
    return PartSpec("attention",
                    {"n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "scale": m.scale, "window": m.window,
                     "keep_first": m.keep_first, "position": position, "values": "keys", "qk_norm": {"eps": cfg.eps},
                     "sink": True,
                     "tensors": {"q": "q", "k": "k", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}}, prefix)


def _feed_forward(mlp, prefix):
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"intermediate_size": mlp.ff, "activation": "silu", "tensors": ("gate", "up", "down")}, prefix)
    return PartSpec("routed_experts",
                    {"n_experts": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff, "activation": "silu",
                     "router_bias": False, "scoring": "softmax_all",
                     "groups": (mlp.groups, mlp.keep_groups) if mlp.groups else None, "shared": None,
                     "tensors": {"expert": "e{e}.{m}", "router": "router"}}, prefix)


def build_zemezen_spec(cfg: ZemezenConfig) -> ModelSpec:
    layers, place = [], {}                                     # place: config layer -> index among the layers that own weights
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        parts = [LayerPart("norm", "norm", _norm(cfg, p + "norm1")),
                 LayerPart("mixer", "mixer", _mixer(cfg, layer, p + "mix."))]
        if layer.mlp is not None:
            parts.append(LayerPart("feed_forward", "feed_forward", _feed_forward(layer.mlp, p + "mlp.")))
        place[i] = len(layers)
        layers.append(LayerSpec("parallel", tuple(parts)))
    # one execution per configured layer, each with a cache of its own; a layer without tensors runs its owner's parts
    schedule = tuple(ScheduleEntry(place[layer.weights_of if layer.weights_of is not None else i])
                     for i, layer in enumerate(cfg.layers))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=cfg.positions(),
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "tensor": "embed", "init_std": 0.5}, ""),
        layers=tuple(layers),
        schedule=schedule,
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "tensor": ""}, "head"),
        stop_token_ids=tuple(cfg.eos_token_id),
        bos_token_id=cfg.bos_token_id)


register_architecture("Zemezen", ZemezenConfig, build_zemezen_spec, model_types=("zemezen",))
