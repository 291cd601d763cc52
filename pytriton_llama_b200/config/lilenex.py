"""Typed configuration of the Lilenex decoder, read from its config.json.

A Lilenex model is a list of layers of two types.  ``attention`` is grouped-query softmax attention
with an RMS norm over the whole query and key projections, a rotation of neighbouring pairs on the
first ``rot.dims`` entries of every head (optionally with YaRN-scaled frequencies), a sliding
window that always keeps the first tokens of the sequence, and optionally the keys and values of
an earlier layer (``kv_from``).  ``gla`` is gated linear attention with one decay per key channel.
A layer's feed-forward is dense (gelu), a routed mixture of gated experts with a shared expert, or
absent.  The residual stream may be kept in several copies that every sub-layer reads as a
weighted sum and writes through a small mixing matrix (``streams``).  Keys of the file:

    architecture, vocab, width, norm.eps, residual_mult, streams,
    layers[i].type, layers[i].mixer.{...}, layers[i].mlp (null, or {kind: dense, ff}, or
    {kind: moe, expert.ff, router.experts, router.top, shared.ff})
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple, Union

from .llama import ConfigError
from .tibepel import _need, _positive_int


def _optional_int(d, key, where, default=0) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if v is None:
        return default
    if isinstance(v, bool) or int(v) != v or int(v) < 0:
        raise ConfigError(f"{where}{key} must be a non-negative integer, got {v!r}")
    return int(v)


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float

    @classmethod
    def from_dict(cls, d, where) -> Optional["YarnScaling"]:
        if d is None:
            return None
        s = cls(*(float(_need(d, k, where)) for k in ("factor", "original", "fast", "slow")))
        if not (s.factor > 0 and s.original > 0 and s.fast > 0 and s.slow > 0):
            raise ConfigError(f"{where}factor, original, fast and slow must be positive")
        return s

    def to_dict(self):
        return {"factor": self.factor, "fast": self.fast, "original": self.original, "slow": self.slow}


@dataclass(frozen=True)
class PairRotation:
    dims: int
    base: float
    scaling: Optional[YarnScaling]

    @classmethod
    def from_dict(cls, d, where, head_dim) -> Optional["PairRotation"]:
        if d is None:
            return None
        dims = _positive_int(d, "dims", where)
        if dims % 2 or dims > head_dim:
            raise ConfigError(f"{where}dims={dims} must be even and at most the head size {head_dim}")
        base = float(_need(d, "base", where))
        if not base > 1:
            raise ConfigError(f"{where}base must be above 1, got {base}")
        return cls(dims, base, YarnScaling.from_dict(d.get("scaling"), where + "scaling."))

    def to_dict(self):
        return {"base": self.base, "dims": self.dims, **({"scaling": self.scaling.to_dict()} if self.scaling else {})}


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                 # 0: every earlier position is seen
    keep_first: int             # positions below this are always seen
    rot: Optional[PairRotation]
    kv_from: Optional[int]      # the layer whose keys and values this one reads instead of its own

    @classmethod
    def from_dict(cls, d, where) -> "AttentionMixerConfig":
        heads, kv = _positive_int(d, "heads", where), _positive_int(d, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"{where}heads={heads} is no multiple of kv_heads={kv}")
        dim = _positive_int(d, "dim", where)
        mask = d.get("mask") or {}
        src = d.get("kv_from")
        if src is not None and (isinstance(src, bool) or int(src) != src or int(src) < 0):
            raise ConfigError(f"{where}kv_from must name a layer, got {src!r}")
        return cls(heads, kv, dim, _positive_int(d, "vdim", where), float(_need(d, "scale", where)),
                   _optional_int(mask, "size", where + "mask."), _optional_int(mask, "keep_first", where + "mask."),
                   PairRotation.from_dict(d.get("rot"), where + "rot.", dim), None if src is None else int(src))

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window:
            d["mask"] = {"keep_first": self.keep_first, "size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class GlaMixerConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int = 0           # inner size of the decay projection for weights drawn at random (0: 16); a checkpoint's tensors say their own

    @classmethod
    def from_dict(cls, d, where) -> "GlaMixerConfig":
        tau = float(_need(d, "tau", where))
        if not tau > 0:
            raise ConfigError(f"{where}tau must be positive, got {tau}")
        return cls(_positive_int(d, "heads", where), _positive_int(d, "dim", where), _positive_int(d, "vdim", where), tau,
                   _optional_int(d, "rank", where))

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "tau": self.tau, "vdim": self.vdim}
        if self.rank:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class MoeMlpConfig:
    ff: int
    experts: int
    top: int
    shared_ff: int          # 0: no shared expert

    def to_dict(self):
        d = {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


def _mlp_from_dict(d, where):
    if d is None:
        return None
    kind = _need(d, "kind", where)
    if kind == "dense":
        return DenseMlpConfig(_positive_int(d, "ff", where))
    if kind == "moe":
        router = _need(d, "router", where)
        experts, top = _positive_int(router, "experts", where + "router."), _positive_int(router, "top", where + "router.")
        if top > experts:
            raise ConfigError(f"{where}router.top={top} exceeds router.experts={experts}")
        shared = d.get("shared")
        return MoeMlpConfig(_positive_int(_need(d, "expert", where), "ff", where + "expert."), experts, top,
                            _positive_int(shared, "ff", where + "shared.") if shared else 0)
    raise ConfigError(f"{where}kind={kind!r} is not supported (known: dense, moe)")


@dataclass(frozen=True)
class LilenexLayerConfig:
    type: str
    mixer: Union[AttentionMixerConfig, GlaMixerConfig]
    mlp: Union[None, DenseMlpConfig, MoeMlpConfig]

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


_MIXERS = {"attention": AttentionMixerConfig, "gla": GlaMixerConfig}


@dataclass(frozen=True)
class LilenexConfig:
    vocab: int
    width: int
    layers: Tuple[LilenexLayerConfig, ...]
    norm_eps: float
    residual_mult: float
    streams: int                    # 0: one stream with a plain residual sum
    initializer_range: float = 0.02
    eos_token_id: Union[None, int, List[int]] = None

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "LilenexConfig":
        raw_layers = _need(data, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]."
            kind = _need(L, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}type={kind!r} is not supported (known: {sorted(_MIXERS)})")
            layers.append(LilenexLayerConfig(kind, _MIXERS[kind].from_dict(_need(L, "mixer", where), where + "mixer."),
                                             _mlp_from_dict(L.get("mlp"), where + "mlp.")))
        for i, L in enumerate(layers):
            src = getattr(L.mixer, "kv_from", None)
            if src is None:
                continue
            where = f"layers[{i}].mixer."
            if src >= i or layers[src].type != "attention" or layers[src].mixer.kv_from is not None:
                raise ConfigError(f"{where}kv_from={src} must name an earlier attention layer that has keys and values of its own")
            a, b = L.mixer, layers[src].mixer
            if (a.kv_heads, a.dim, a.vdim) != (b.kv_heads, b.dim, b.vdim):
                raise ConfigError(f"{where}kv_heads, dim and vdim must equal those of layer {src}")
        eps = float(_need(_need(data, "norm", ""), "eps", "norm."))
        if not eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        eos = data.get("eos_token_id")
        return cls(vocab=_positive_int(data, "vocab", ""), width=_positive_int(data, "width", ""), layers=tuple(layers),
                   norm_eps=eps, residual_mult=float(data.get("residual_mult", 1.0)),
                   streams=_optional_int(data, "streams", ""),
                   initializer_range=float(data.get("initializer_range", 0.02)),
                   eos_token_id=[int(e) for e in eos] if isinstance(eos, (list, tuple)) else eos)

    @classmethod
    def from_folder(cls, folder: Union[str, Path]) -> "LilenexConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": "Lilenex", "layers": [L.to_dict() for L in self.layers], "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width,
             "initializer_range": self.initializer_range}
        if self.streams:
            d["streams"] = self.streams
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    @property
    def eos_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        return [self.eos_token_id] if isinstance(self.eos_token_id, int) else list(self.eos_token_id)
