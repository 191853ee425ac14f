"""Typed configuration of the Zamizen architecture, read from config.json.

config.json names the architecture by an `architecture` string and lists the layers one by one: each entry gives its
`type` (which mixer: `attention` or `latent_attention`), the mixer's sizes (`mixer`) and its feed-forward (`mlp`, or
null for none).  Every size and every constant that can differ between two models of the design is read from there;
nothing is assumed equal between layers.  A value of the wrong kind, a missing size and an unknown mixer or
feed-forward kind are refused by name; keys this reader does not know are kept in `ignored` and have no effect.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, _is_int

MIXER_TYPES = ("attention", "latent_attention")


def _int(d: Dict[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if not _is_int(v) or v < minimum:
        raise ConfigError(f"zamizen: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return int(v)


def _real(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"zamizen: {where}.{key} must be a finite number, got {v!r}")
    return float(v)


def _positive(d: Dict[str, Any], key: str, where: str) -> float:
    v = _real(d, key, where)
    if not v > 0:
        raise ConfigError(f"zamizen: {where}.{key} must be positive, got {v!r}")
    return v


def _obj(d: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"zamizen: {where}.{key} must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class RotScaling:
    """Frequencies blended for contexts longer than `original` positions (see parts.rope.blended_frequencies)."""
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self) -> Dict[str, Any]:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}

    def as_tuple(self) -> Tuple[float, float, float, float]:
        return (self.factor, self.original, self.fast, self.slow)


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    conv: int = 1                       # taps of the causal filter on q, k and v (1: none)
    kv_from: Optional[int] = None       # the layer whose keys and values this one reads instead of making its own

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.conv > 1:
            d["conv"] = self.conv
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotScaling] = None

    def to_dict(self) -> Dict[str, Any]:
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_scaling is not None:
            rot["scaling"] = self.rot_scaling.to_dict()
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, "rot": rot}


@dataclass(frozen=True)
class ZamizenLayer:
    type: str
    mixer: Any
    mlp: Optional[DenseMlp]

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


def _read_rot(m: Dict[str, Any], where: str, limit: int, what: str):
    """(base, dims) of a mixer's `rot` object; `rot` may be missing when nothing is rotated."""
    rot = m.get("rot")
    if rot is None:
        return 10000.0, 0, None                      # nothing is rotated: the base is never used
    rot = _obj(m, "rot", where)
    dims = _int(rot, "dims", where + ".rot", minimum=0)
    if dims % 2 or dims > limit:
        raise ConfigError(f"zamizen: {where}.rot.dims must be even and at most {what} ({limit}), got {dims}")
    return (_positive(rot, "base", where + ".rot") if dims else 10000.0), dims, rot


def _read_mixer(kind: str, m: Dict[str, Any], where: str):
    if kind == "attention":
        heads, kv_heads, dim = _int(m, "heads", where), _int(m, "kv_heads", where), _int(m, "dim", where)
        if heads % kv_heads:
            raise ConfigError(f"zamizen: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        base, dims, _ = _read_rot(m, where, dim, "dim")
        conv = _int(m, "conv", where) if m.get("conv") is not None else 1
        kv_from = _int(m, "kv_from", where, minimum=0) if m.get("kv_from") is not None else None
        return AttentionMixer(heads, kv_heads, dim, _int(m, "vdim", where), _real(m, "scale", where), base, dims, conv, kv_from)
    if kind == "latent_attention":
        rot_dim = _int(m, "rot_dim", where, minimum=0)
        base, dims, rot = _read_rot(m, where, rot_dim, "rot_dim")
        scaling = None
        if rot is not None and rot.get("scaling") is not None:
            s, w = _obj(rot, "scaling", where + ".rot"), where + ".rot.scaling"
            scaling = RotScaling(_positive(s, "factor", w), _positive(s, "original", w), _positive(s, "fast", w), _positive(s, "slow", w))
        return LatentMixer(_int(m, "heads", where), _int(m, "dim", where), rot_dim, _int(m, "vdim", where), _int(m, "kv_rank", where),
                           _real(m, "scale", where), base, dims, scaling)
    raise ConfigError(f"zamizen: {where}: mixer type {kind!r} is not one of {list(MIXER_TYPES)}")


@dataclass(frozen=True)
class ZamizenConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[ZamizenLayer, ...]
    norm_eps: float
    residual_mult: float = 1.0
    ignored: Tuple[str, ...] = field(default=(), compare=False)

    model_type = "zamizen"
    class_name = "Zamizen"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ZamizenConfig":
        if raw.get("architecture") != "Zamizen":
            raise ConfigError(f"zamizen: config.json names architecture {raw.get('architecture')!r}")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("zamizen: layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"zamizen: {where} must be an object")
            kind = entry.get("type")
            mixer = _read_mixer(kind, _obj(entry, "mixer", where), where + ".mixer")
            mlp_raw = entry.get("mlp")
            mlp = None
            if mlp_raw is not None:
                if not isinstance(mlp_raw, dict):
                    raise ConfigError(f"zamizen: {where}.mlp must be an object or null")
                if mlp_raw.get("kind") != "dense":
                    raise ConfigError(f"zamizen: {where}.mlp.kind {mlp_raw.get('kind')!r} is not supported (\"dense\")")
                mlp = DenseMlp(_int(mlp_raw, "ff", where + ".mlp"))
            layers.append(ZamizenLayer(kind, mixer, mlp))
        # A layer that reads another's keys and values names an earlier attention layer of the same geometry that makes its own.
        for i, layer in enumerate(layers):
            m = layer.mixer
            if isinstance(m, AttentionMixer) and m.kv_from is not None:
                where = f"layers[{i}].mixer.kv_from"
                if m.kv_from >= i:
                    raise ConfigError(f"zamizen: {where} must name an earlier layer, got {m.kv_from}")
                src = layers[m.kv_from].mixer
                if not isinstance(src, AttentionMixer) or src.kv_from is not None:
                    raise ConfigError(f"zamizen: {where} names layer {m.kv_from}, which has no keys and values of its own")
                if (src.kv_heads, src.dim, src.vdim) != (m.kv_heads, m.dim, m.vdim):
                    raise ConfigError(f"zamizen: {where}: layer {m.kv_from} has other key/value heads or widths")
        norm = _obj(raw, "norm", "config")
        eps = _real(norm, "eps", "norm")
        if not eps >= 0:
            raise ConfigError("zamizen: norm.eps must not be negative")
        mult = _real(raw, "residual_mult", "config") if raw.get("residual_mult") is not None else 1.0
        known = {"architecture", "layers", "norm", "residual_mult", "vocab", "width", "torch_dtype"}
        return cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"), layers=tuple(layers), norm_eps=eps,
                   residual_mult=mult, ignored=tuple(sorted(k for k in raw if k not in known)))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": "Zamizen", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "layers": [layer.to_dict() for layer in self.layers]}
