"""Typed configuration of the Zemezen decoder, read from config.json's own keys.

config.json of this architecture is nested: ``layers`` lists the layers in order, each with its ``type``
("channel_delta", "latent_attention" or "attention"), the mixer's sizes (``mixer``) and its feed-forward (``mlp``:
``kind`` "dense" with ``ff``, or "moe" with ``expert`` {ff} and ``router`` {experts, top, groups {count, keep}};
null: none).  A layer with ``weights_of`` j owns no tensors and runs with layer j's, on a cache of its own.
``norm.eps`` is every norm's eps; ``vocab`` and ``width`` the global sizes.  The design states no position limit:
``max_positions`` is an optional key.  Every size and constant is taken from there; nothing is assumed about
their values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError
from .kubedra import _get

MIXER_TYPES = ("channel_delta", "latent_attention", "attention")
DEFAULT_MAX_POSITIONS = 65536


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int                    # value heads (one state each)
    kv_heads: int                 # query/key heads
    dim: int                      # key channels per head
    vdim: int                     # value channels per head
    conv: int                     # taps of the short convolution
    ranks: Optional[tuple] = None         # (decay, gate): only the random-weights mode needs them

    @classmethod
    def from_dict(cls, d, where):
        ranks = d.get("ranks")
        heads = _get(d, "heads", int, where)
        return cls(heads, _get(d, "kv_heads", int, where, default=heads, required=False), _get(d, "dim", int, where),
                   _get(d, "vdim", int, where), _get(d, "conv", int, where),
                   (int(ranks[0]), int(ranks[1])) if ranks else None)

    def to_dict(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.ranks is not None:
            out["ranks"] = list(self.ranks)
        return out

    def check(self, where):
        if min(self.heads, self.kv_heads, self.dim, self.vdim, self.conv) <= 0 or self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float

    @classmethod
    def from_dict(cls, d, where):
        return cls(_get(d, "heads", int, where), _get(d, "dim", int, where), _get(d, "vdim", int, where),
                   _get(d, "kv_rank", int, where), _get(d, "scale", float, where))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale}

    def check(self, where):
        if min(self.heads, self.dim, self.vdim, self.kv_rank) <= 0:
            raise ConfigError(f"config.json: {where}: sizes must be positive")


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int                     # the values are the keys: equal to dim
    scale: float
    window: Optional[int]         # mask.size; None (no mask in the entry): every earlier key
    keep_first: int               # mask.keep_first
    rot_dims: int
    rot_base: float

    @classmethod
    def from_dict(cls, d, where):
        mask, rot = d.get("mask"), d.get("rot")
        dim = _get(d, "dim", int, where)
        return cls(_get(d, "heads", int, where), _get(d, "kv_heads", int, where), dim,
                   _get(d, "vdim", int, where, default=dim, required=False), _get(d, "scale", float, where),
                   _get(mask, "size", int, where + ".mask", required=mask is not None),
                   _get(mask, "keep_first", int, where + ".mask", default=0, required=False),
                   _get(rot, "dims", int, where + ".rot", default=0, required=rot is not None),
                   _get(rot, "base", float, where + ".rot", default=10000.0, required=rot is not None))

    def to_dict(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window, "keep_first": self.keep_first}
        out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        return out

    def check(self, where):
        if min(self.heads, self.kv_heads, self.dim) <= 0 or self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
        if self.vdim != self.dim:
            raise ConfigError(f"config.json: {where}: the values are the keys, so vdim {self.vdim} must equal dim {self.dim}")
        if (self.window is not None and self.window < 1) or self.keep_first < 0 or (self.keep_first and self.window is None):
            raise ConfigError(f"config.json: {where}.mask: a window holds at least the token itself, keep_first is not negative")
        if self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.dim or self.rot_base <= 0:
            raise ConfigError(f"config.json: {where}.rot: dims must be even and at most dim, base positive")


_MIXERS = {"channel_delta": DeltaMixerConfig, "latent_attention": LatentMixerConfig, "attention": AttentionMixerConfig}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                             # "dense" or "moe"
    ff: int                               # dense: the hidden width; moe: one expert's
    experts: int = 0
    top: int = 0
    groups: int = 0                       # 0: every expert can be chosen
    keep_groups: int = 0

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "kind", str, where)
        if kind == "dense":
            return cls("dense", _get(d, "ff", int, where))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind = {kind!r}; known: 'dense', 'moe'")
        expert, router = d.get("expert"), d.get("router")
        groups = router.get("groups") if isinstance(router, dict) else None
        cfg = cls("moe", _get(expert, "ff", int, where + ".expert"), _get(router, "experts", int, where + ".router"),
                  _get(router, "top", int, where + ".router"),
                  _get(groups, "count", int, where + ".router.groups") if groups else 0,
                  _get(groups, "keep", int, where + ".router.groups") if groups else 0)
        if not 0 < cfg.top <= cfg.experts:
            raise ConfigError(f"config.json: {where}.router cannot choose {cfg.top} of {cfg.experts} experts")
        if cfg.groups and (cfg.groups < 0 or cfg.experts % cfg.groups or not 0 < cfg.keep_groups <= cfg.groups
                           or cfg.top > cfg.keep_groups * (cfg.experts // cfg.groups)):
            raise ConfigError(f"config.json: {where}.router.groups: {cfg.experts} experts in {cfg.groups} groups of which "
                              f"{cfg.keep_groups} stay cannot give {cfg.top} choices")
        return cfg

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top}
        if self.groups:
            router["groups"] = {"count": self.groups, "keep": self.keep_groups}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": router}


@dataclass(frozen=True)
class ZemezenLayerConfig:
    type: str
    mixer: object
    mlp: Optional[FeedForwardConfig]
    weights_of: Optional[int] = None

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "type", str, where)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}.type = {kind!r}; known: {list(MIXER_TYPES)}")
        if not isinstance(d.get("mixer"), dict):
            raise ConfigError(f"config.json: {where} lacks its mixer's sizes")
        mixer = _MIXERS[kind].from_dict(d["mixer"], where + ".mixer")
        mixer.check(where + ".mixer")
        mlp = FeedForwardConfig.from_dict(d["mlp"], where + ".mlp") if d.get("mlp") else None
        return cls(kind, mixer, mlp, _get(d, "weights_of", int, where, required=False))

    def to_dict(self):
        out = {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}
        if self.weights_of is not None:
            out["weights_of"] = self.weights_of
        return out


@dataclass(frozen=True)
class ZemezenConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple                         # of ZemezenLayerConfig
    max_positions: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: tuple = ()
    architecture: str = "Zemezen"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks its list of layers")
        parsed = tuple(ZemezenLayerConfig.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(layers))
        for i, layer in enumerate(parsed):
            j = layer.weights_of
            if j is None:
                continue
            if not 0 <= j < len(parsed) or j == i or parsed[j].weights_of is not None:
                raise ConfigError(f"config.json: layers[{i}].weights_of = {j} must name another layer that owns its weights")
            if (parsed[j].type, parsed[j].mixer, parsed[j].mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"config.json: layers[{i}] runs with the weights of layer {j} but differs from it")
        eos = d.get("eos_token_id")
        eos = () if eos is None else tuple(int(t) for t in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cfg = cls(_get(d, "vocab", int, "config"), _get(d, "width", int, "config"), _get(d.get("norm"), "eps", float, "norm"),
                  parsed, _get(d, "max_positions", int, "config", required=False),
                  _get(d, "bos_token_id", int, "config", required=False), eos)
        if min(cfg.vocab, cfg.width) <= 0 or cfg.eps <= 0 or (cfg.max_positions is not None and cfg.max_positions <= 0):
            raise ConfigError("config.json: vocab, width, norm.eps and max_positions must be positive")
        return cfg

    def to_dict(self):
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.max_positions is not None:
            out["max_positions"] = self.max_positions
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out

    def positions(self):
        return self.max_positions or DEFAULT_MAX_POSITIONS
