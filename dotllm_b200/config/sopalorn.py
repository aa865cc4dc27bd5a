"""Typed configuration of the Sopalorn decoder, read from config.json's own keys.

config.json of this architecture is nested: ``layers`` lists the layers in order, each with its ``type`` ("attention",
"lightning" or "parallel"), the mixer's sizes (``mixer``; a parallel layer's has ``left`` and ``right``) and its feed-forward
(``mlp``: ``kind`` "dense" with ``ff`` and ``limit``, or "moe" with ``expert`` {ff} and ``router`` {experts, identity, top,
scale}; null: none).  An attention mixer with ``kv_from`` j has no keys and values of its own and reads layer j's.
``embedding.scale`` multiplies the embedding, ``logit_scale`` the logits, ``norm.eps`` is every norm's eps, ``streams`` the
number of copies the residual stream is kept in (absent: one stream and the plain residual sum), ``vocab`` and ``width`` the
global sizes.  The design states no position limit: ``max_positions`` is an optional key.  Every size and constant is
taken from there; nothing is assumed about their values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError
from .kubedra import _get

MIXER_TYPES = ("attention", "lightning", "parallel")
DEFAULT_MAX_POSITIONS = 65536


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    scaling: Optional[tuple] = None       # (factor, original, fast, slow)

    @classmethod
    def from_dict(cls, d, where):
        sc = d.get("scaling")
        scaling = None
        if sc:
            scaling = tuple(_get(sc, key, float, where + ".scaling") for key in ("factor", "original", "fast", "slow"))
        cfg = cls(_get(d, "dims", int, where), _get(d, "base", float, where), scaling)
        if cfg.dims < 0 or cfg.dims % 2 or cfg.base <= 0 or (scaling and (scaling[0] <= 0 or scaling[1] <= 0)):
            raise ConfigError(f"config.json: {where}: dims must be even, base and the scaling's factor and length positive")
        return cfg

    def to_dict(self):
        out = {"dims": self.dims, "base": self.base}
        if self.scaling:
            factor, original, fast, slow = self.scaling
            out["scaling"] = {"factor": factor, "original": int(original) if float(original).is_integer() else original,
                              "fast": fast, "slow": slow}
        return out


@dataclass(frozen=True)
class AttentionConfig:
    """Softmax attention with grouped key/value heads.  In an "attention" layer: a norm over the whole query and the whole
    key projection, a rotation, one added to the softmax's denominator, maybe another layer's keys and values.  As the left
    side of a "parallel" layer: no norm, no rotation, a sliding window, a learned sink per head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None          # mask.size; None: every earlier key
    rot: Optional[RotationConfig] = None
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, d, where):
        mask, rot = d.get("mask"), d.get("rot")
        cfg = cls(_get(d, "heads", int, where), _get(d, "kv_heads", int, where), _get(d, "dim", int, where),
                  _get(d, "vdim", int, where), _get(d, "scale", float, where),
                  _get(mask, "size", int, where + ".mask") if mask else None,
                  RotationConfig.from_dict(rot, where + ".rot") if rot else None,
                  _get(d, "kv_from", int, where, required=False))
        if min(cfg.heads, cfg.kv_heads, cfg.dim, cfg.vdim) <= 0 or cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
        if cfg.window is not None and cfg.window < 1:
            raise ConfigError(f"config.json: {where}.mask: a window holds at least the token itself")
        if cfg.rot is not None and cfg.rot.dims > cfg.dim:
            raise ConfigError(f"config.json: {where}.rot: {cfg.rot.dims} rotated channels in a head of {cfg.dim}")
        return cfg

    def to_dict(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple                          # one constant per head

    @classmethod
    def from_dict(cls, d, where):
        decay = d.get("decay")
        if not isinstance(decay, (list, tuple)):
            raise ConfigError(f"config.json: {where} lacks its list of decays")
        cfg = cls(_get(d, "heads", int, where), _get(d, "dim", int, where), _get(d, "vdim", int, where),
                  tuple(float(x) for x in decay))
        if min(cfg.heads, cfg.dim, cfg.vdim) <= 0 or len(cfg.decay) != cfg.heads or not all(0.0 <= x <= 1.0 for x in cfg.decay):
            raise ConfigError(f"config.json: {where}: sizes must be positive, with one decay in [0, 1] per head")
        return cfg

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class DeltaConfig:
    heads: int                    # value heads (one state each)
    kv_heads: int                 # query/key heads
    dim: int
    vdim: int
    conv: int                     # taps of the short convolutions

    @classmethod
    def from_dict(cls, d, where):
        heads = _get(d, "heads", int, where)
        cfg = cls(heads, _get(d, "kv_heads", int, where, default=heads, required=False), _get(d, "dim", int, where),
                  _get(d, "vdim", int, where), _get(d, "conv", int, where))
        if min(cfg.heads, cfg.kv_heads, cfg.dim, cfg.vdim, cfg.conv) <= 0 or cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
        return cfg

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class ParallelConfig:
    left: AttentionConfig
    right: DeltaConfig

    @classmethod
    def from_dict(cls, d, where):
        if not isinstance(d.get("left"), dict) or not isinstance(d.get("right"), dict):
            raise ConfigError(f"config.json: {where} lacks its left or right mixer")
        left = AttentionConfig.from_dict(d["left"], where + ".left")
        if left.kv_from is not None or left.rot is not None:
            raise ConfigError(f"config.json: {where}.left: the attention beside a recurrence has keys of its own and no rotation")
        return cls(left, DeltaConfig.from_dict(d["right"], where + ".right"))

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


_MIXERS = {"attention": AttentionConfig, "lightning": LightningConfig, "parallel": ParallelConfig}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                             # "dense" or "moe"
    ff: int                               # dense: the hidden width; moe: one expert's
    limit: float = 0.0                    # dense: the clamp of gate and up (0, or no key: none)
    experts: int = 0                      # experts with matrices
    identity: int = 0                     # experts without: they give back their input
    top: int = 0
    scale: float = 1.0                    # on the chosen experts' normalised weights

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "kind", str, where)
        if kind == "dense":
            cfg = cls("dense", _get(d, "ff", int, where), _get(d, "limit", float, where, default=0.0, required=False))
            if cfg.ff <= 0 or cfg.limit < 0:
                raise ConfigError(f"config.json: {where}: ff must be positive and limit not negative")
            return cfg
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind = {kind!r}; known: 'dense', 'moe'")
        expert, router = d.get("expert"), d.get("router")
        cfg = cls("moe", _get(expert, "ff", int, where + ".expert"), 0.0, _get(router, "experts", int, where + ".router"),
                  _get(router, "identity", int, where + ".router", default=0, required=False),
                  _get(router, "top", int, where + ".router"), _get(router, "scale", float, where + ".router", default=1.0, required=False))
        if cfg.ff <= 0 or cfg.experts <= 0 or cfg.identity < 0 or not 0 < cfg.top <= cfg.experts + cfg.identity:
            raise ConfigError(f"config.json: {where}.router cannot choose {cfg.top} of {cfg.experts} + {cfg.identity} experts")
        return cfg

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff, **({"limit": self.limit} if self.limit else {})}
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "identity": self.identity, "top": self.top, "scale": self.scale}}


@dataclass(frozen=True)
class SopalornLayerConfig:
    type: str
    mixer: object
    mlp: Optional[FeedForwardConfig]

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "type", str, where)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}.type = {kind!r}; known: {list(MIXER_TYPES)}")
        if not isinstance(d.get("mixer"), dict):
            raise ConfigError(f"config.json: {where} lacks its mixer's sizes")
        mixer = _MIXERS[kind].from_dict(d["mixer"], where + ".mixer")
        mlp = FeedForwardConfig.from_dict(d["mlp"], where + ".mlp") if d.get("mlp") else None
        return cls(kind, mixer, mlp)

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class SopalornConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple                         # of SopalornLayerConfig
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    streams: Optional[int] = None         # None: one stream, the plain residual sum
    max_positions: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: tuple = ()
    architecture: str = "Sopalorn"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks its list of layers")
        parsed = tuple(SopalornLayerConfig.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(layers))
        for i, layer in enumerate(parsed):
            j = layer.mixer.kv_from if layer.type == "attention" else None
            if j is None:
                continue
            # the keys a layer borrows must exist when it runs, and fit its queries
            if not 0 <= j < i or parsed[j].type != "attention" or parsed[j].mixer.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {j} must name an earlier attention layer with keys of its own")
            a, b = layer.mixer, parsed[j].mixer
            if (a.kv_heads, a.dim, a.vdim, a.rot, a.window) != (b.kv_heads, b.dim, b.vdim, b.rot, b.window):
                raise ConfigError(f"config.json: layers[{i}] reads the keys and values of layer {j}, whose heads, widths, rotation or window differ")
        eos = d.get("eos_token_id")
        eos = () if eos is None else tuple(int(t) for t in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cfg = cls(_get(d, "vocab", int, "config"), _get(d, "width", int, "config"), _get(d.get("norm"), "eps", float, "norm"), parsed,
                  _get(d.get("embedding"), "scale", float, "embedding", default=1.0, required=False),
                  _get(d, "logit_scale", float, "config", default=1.0, required=False),
                  _get(d, "streams", int, "config", required=False), _get(d, "max_positions", int, "config", required=False),
                  _get(d, "bos_token_id", int, "config", required=False), eos)
        if min(cfg.vocab, cfg.width) <= 0 or cfg.eps <= 0 or (cfg.max_positions is not None and cfg.max_positions <= 0) \
                or (cfg.streams is not None and cfg.streams <= 0):
            raise ConfigError("config.json: vocab, width, norm.eps, streams and max_positions must be positive")
        return cfg

    def to_dict(self):
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.max_positions is not None:
            out["max_positions"] = self.max_positions
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out

    def positions(self):
        return self.max_positions or DEFAULT_MAX_POSITIONS
