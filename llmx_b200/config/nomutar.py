"""Typed configuration of the Nomutar architecture, read from config.json.

config.json names the architecture by an `architecture` string and lists the layers one by one: each entry gives its
`type` (which of three softmax-attention mixers), the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`:
a dense gated unit, a routed mixture of experts, or null for none).  `loop` runs a stretch of layers several times with
the same weights, `canon` gives the taps of the causal filter on every mixer's input, `norm` the norm's epsilon and its
number of groups, `embedding` a factor and the hashed pair table.  Every size and every constant that can differ between
two models of the design is read from there; nothing is assumed equal between layers, and what config.json does not
mention is not there (no window, no cap, no filter, no loop).  A value of the wrong kind, a missing size and an unknown
mixer or feed-forward kind are refused by name; keys this reader does not know are kept in `ignored` and have no effect.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, _is_int

MIXER_TYPES = ("attention", "attention_2", "attention_3")


def _int(d: Dict[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if not _is_int(v) or v < minimum:
        raise ConfigError(f"nomutar: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return int(v)


def _real(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"nomutar: {where}.{key} must be a finite number, got {v!r}")
    return float(v)


def _positive(d: Dict[str, Any], key: str, where: str) -> float:
    v = _real(d, key, where)
    if not v > 0:
        raise ConfigError(f"nomutar: {where}.{key} must be positive, got {v!r}")
    return v


def _obj(d: Dict[str, Any], key: str, where: str) -> Dict[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"nomutar: {where}.{key} must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class RotScaling:
    """How the rotation's frequencies are changed for long contexts.  `kind` "bands": wavelengths shorter than
    original / high keep their frequency, longer than original / low take f / factor, those between are blended
    (parts.rope.banded_frequencies).  `kind` "ramp": a ramp over the pair index between the pairs that make `fast` and
    `slow` turns in `original` positions, and a factor on cosines and sines (parts.rope.blended_frequencies)."""
    kind: str
    factor: float
    original: float
    a: float            # bands: low;  ramp: fast
    b: float            # bands: high; ramp: slow

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "bands":
            return {"factor": self.factor, "low": self.a, "high": self.b, "original": self.original}
        return {"factor": self.factor, "original": self.original, "fast": self.a, "slow": self.b}


@dataclass(frozen=True)
class AttentionMixer:
    """One of the three mixers.  What the `type` fixes: `attention`: one RMS norm over all queries and one over all keys,
    rotation in the two-halves pairing, values rotated by their position and outputs turned back, a learned sink per head;
    `attention_2`: biases on q, k and v, rotation of neighbouring pairs, a sink of zero; `attention_3`: the norms of
    `attention`, two-halves pairing, causal over everything, plain softmax."""
    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float = 10000.0
    rot_dims: int = 0
    rot_scaling: Optional[RotScaling] = None
    window: Optional[int] = None
    softcap: Optional[float] = None

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_dims or self.type == "attention":
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_scaling is not None:
                d["rot"]["scaling"] = self.rot_scaling.to_dict()
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        return d


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class RoutedMlp:
    """`experts` gated units of width `ff`, `top` of them a token, chosen by a router; a shared unit of width `shared_ff`
    beside them (times a sigmoid gate of its own), or none."""
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class NomutarLayer:
    mixer: AttentionMixer
    mlp: Any                       # DenseMlp, RoutedMlp or None

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.mixer.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class Loop:
    """Layers start .. stop-1 run `times` times in a row with the same weights."""
    start: int = 0
    stop: int = 0
    times: int = 1

    def to_dict(self) -> Dict[str, Any]:
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class PairTable:
    """The hashed table of token pairs: row (token before * mul_prev + token * mul_cur) mod buckets; row `buckets` for a
    request's first token."""
    buckets: int
    mul_prev: int
    mul_cur: int

    def to_dict(self) -> Dict[str, Any]:
        return {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}


def _read_scaling(raw: Any, where: str) -> Optional[RotScaling]:
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"nomutar: {where} must be an object or null")
    factor, original = _positive(raw, "factor", where), _positive(raw, "original", where)
    if "low" in raw or "high" in raw:
        low, high = _positive(raw, "low", where), _positive(raw, "high", where)
        if not high > low:
            raise ConfigError(f"nomutar: {where}.high must exceed low")
        return RotScaling("bands", factor, original, low, high)
    if "fast" in raw or "slow" in raw:
        return RotScaling("ramp", factor, original, _positive(raw, "fast", where), _positive(raw, "slow", where))
    raise ConfigError(f"nomutar: {where} names neither low / high nor fast / slow")


def _read_mixer(kind: Any, m: Dict[str, Any], where: str) -> AttentionMixer:
    if kind not in MIXER_TYPES:
        raise ConfigError(f"nomutar: {where}: mixer type {kind!r} is not one of {list(MIXER_TYPES)}")
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"nomutar: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    dim, vdim = _int(m, "dim", where), _int(m, "vdim", where)
    base, dims, scaling = 10000.0, 0, None
    if m.get("rot") is not None:
        rot = _obj(m, "rot", where)
        dims = _int(rot, "dims", where + ".rot", minimum=0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"nomutar: {where}.rot.dims must be even and at most dim ({dim}), got {dims}")
        base = _positive(rot, "base", where + ".rot")
        scaling = _read_scaling(rot.get("scaling"), where + ".rot.scaling")
    if kind == "attention" and vdim % 2:
        raise ConfigError(f"nomutar: {where}.vdim must be even (the values are rotated in pairs), got {vdim}")
    window = softcap = None
    if kind != "attention_3":
        if m.get("mask") is not None:
            window = _int(_obj(m, "mask", where), "size", where + ".mask")
        if m.get("softcap") is not None:
            softcap = _positive(m, "softcap", where)
    return AttentionMixer(kind, heads, kv_heads, dim, vdim, _real(m, "scale", where), base, dims, scaling, window, softcap)


def _read_mlp(raw: Any, where: str):
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"nomutar: {where} must be an object or null")
    kind = raw.get("kind")
    if kind == "dense":
        return DenseMlp(_int(raw, "ff", where))
    if kind == "moe":
        router = _obj(raw, "router", where)
        experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"nomutar: {where}.router.top ({top}) exceeds the number of experts ({experts})")
        shared_ff = None if raw.get("shared") is None else _int(_obj(raw, "shared", where), "ff", where + ".shared")
        return RoutedMlp(experts, top, _int(_obj(raw, "expert", where), "ff", where + ".expert"), shared_ff)
    raise ConfigError(f"nomutar: {where}.kind {kind!r} is not supported (\"dense\", \"moe\")")


@dataclass(frozen=True)
class NomutarConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[NomutarLayer, ...]
    norm_eps: float
    norm_groups: int = 1
    residual_mult: float = 1.0
    canon_taps: int = 0                  # taps of the causal filter on a mixer's input (0: no filter)
    loop: Loop = Loop()
    embedding_scale: float = 1.0
    pair_table: Optional[PairTable] = None
    logit_softcap: Optional[float] = None
    ignored: Tuple[str, ...] = field(default=(), compare=False)

    model_type = "nomutar"
    class_name = "Nomutar"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "NomutarConfig":
        if raw.get("architecture") != "Nomutar":
            raise ConfigError(f"nomutar: config.json names architecture {raw.get('architecture')!r}")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("nomutar: layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"nomutar: {where} must be an object")
            mixer = _read_mixer(entry.get("type"), _obj(entry, "mixer", where), where + ".mixer")
            layers.append(NomutarLayer(mixer, _read_mlp(entry.get("mlp"), where + ".mlp")))
        width = _int(raw, "width", "config")
        loop = Loop()
        if raw.get("loop") is not None:
            lr = _obj(raw, "loop", "config")
            loop = Loop(_int(lr, "start", "loop", minimum=0), _int(lr, "stop", "loop", minimum=0), _int(lr, "times", "loop"))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"nomutar: loop must have 0 <= start <= stop <= {len(layers)} layers, got {lr!r}")
        norm = _obj(raw, "norm", "config")
        eps = _real(norm, "eps", "norm")
        if not eps >= 0:
            raise ConfigError("nomutar: norm.eps must not be negative")
        groups = _int(norm, "groups", "norm") if "groups" in norm else 1
        if width % groups:
            raise ConfigError(f"nomutar: width ({width}) must be a multiple of norm.groups ({groups})")
        taps = _int(_obj(raw, "canon", "config"), "taps", "canon") if raw.get("canon") is not None else 0
        emb = raw.get("embedding")
        emb_scale, pairs = 1.0, None
        if emb is not None:
            emb = _obj(raw, "embedding", "config")
            if "scale" in emb:
                emb_scale = _real(emb, "scale", "embedding")
            if emb.get("bigram") is not None:
                b = _obj(emb, "bigram", "embedding")
                pairs = PairTable(_int(b, "buckets", "embedding.bigram"), _int(b, "mul_prev", "embedding.bigram", minimum=0),
                                  _int(b, "mul_cur", "embedding.bigram", minimum=0))
        cap = _positive(raw, "logit_softcap", "config") if raw.get("logit_softcap") is not None else None
        mult = _real(raw, "residual_mult", "config") if "residual_mult" in raw else 1.0
        known = {"architecture", "layers", "loop", "norm", "embedding", "logit_softcap", "vocab", "width", "canon", "residual_mult",
                 "torch_dtype"}
        return cls(vocab=_int(raw, "vocab", "config"), width=width, layers=tuple(layers), norm_eps=eps, norm_groups=groups,
                   residual_mult=mult, canon_taps=taps, loop=loop, embedding_scale=emb_scale, pair_table=pairs, logit_softcap=cap,
                   ignored=tuple(sorted(k for k in raw if k not in known)))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": "Nomutar", "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "residual_mult": self.residual_mult,
                             "embedding": {"scale": self.embedding_scale}, "loop": self.loop.to_dict(),
                             "layers": [layer.to_dict() for layer in self.layers]}
        if self.pair_table is not None:
            d["embedding"]["bigram"] = self.pair_table.to_dict()
        if self.canon_taps > 0:
            d["canon"] = {"taps": self.canon_taps}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d

    def layer_runs(self):
        """The layers in the order they run: the looped stretch `times` times in a row, the rest once."""
        n, lp = len(self.layers), self.loop
        runs = list(range(lp.start))
        for _ in range(lp.times if lp.stop > lp.start else 0):
            runs += list(range(lp.start, lp.stop))
        return runs + list(range(lp.stop, n))
