"""Typed configuration of the Tibepel decoder, read from its config.json.

A Tibepel model is a list of layers of two types.  ``mamba1`` has a selective-scan mixer;
``parallel`` runs a chunk-masked attention (distance bias, mixed head weights, normed values)
beside a gated delta rule and adds the two with fixed scales.  Every layer may have a clamped
gated feed-forward and ends with a term looked up by the token itself.  Every size, the order of
the layers and every constant that may differ between models is a key of the file:

    architecture, vocab, width, embedding.scale, norm.eps, logit_softcap, token_side.dim,
    layers[i].type, layers[i].mixer.{...}, layers[i].mlp (null or {kind, ff, limit})
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple, Union

from .llama import ConfigError


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


def _positive_int(d, key, where) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or int(v) != v or int(v) <= 0:
        raise ConfigError(f"{where}{key} must be a positive integer, got {v!r}")
    return int(v)


@dataclass(frozen=True)
class ScanMixerConfig:
    """``mamba1``: selective scan over ``inner`` channels with ``state`` values each."""
    inner: int
    state: int
    dt_rank: int
    conv: int

    @classmethod
    def from_dict(cls, d, where) -> "ScanMixerConfig":
        return cls(*( _positive_int(d, k, where) for k in ("inner", "state", "dt_rank", "conv")))

    def to_dict(self):
        return {"conv": self.conv, "dt_rank": self.dt_rank, "inner": self.inner, "state": self.state}


@dataclass(frozen=True)
class ChunkAttentionConfig:
    """Left member of ``parallel``: grouped-query attention inside blocks of ``mask_size`` positions."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask_size: int

    @classmethod
    def from_dict(cls, d, where) -> "ChunkAttentionConfig":
        heads, kv = _positive_int(d, "heads", where), _positive_int(d, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"{where}heads={heads} is no multiple of kv_heads={kv}")
        mask = _need(d, "mask", where)
        return cls(heads, kv, _positive_int(d, "dim", where), _positive_int(d, "vdim", where),
                   float(_need(d, "scale", where)), _positive_int(mask, "size", where + "mask."))

    def to_dict(self):
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "mask": {"size": self.mask_size},
                "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class DeltaRuleConfig:
    """Right member of ``parallel``: gated delta rule, ``heads`` value heads over ``kv_heads`` query/key heads."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, d, where) -> "DeltaRuleConfig":
        heads, kv = _positive_int(d, "heads", where), _positive_int(d, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"{where}heads={heads} is no multiple of kv_heads={kv}")
        return cls(heads, kv, _positive_int(d, "dim", where), _positive_int(d, "vdim", where), _positive_int(d, "conv", where))

    def to_dict(self):
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: ChunkAttentionConfig
    right: DeltaRuleConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d, where) -> "ParallelMixerConfig":
        return cls(ChunkAttentionConfig.from_dict(_need(d, "left", where), where + "left."),
                   DeltaRuleConfig.from_dict(_need(d, "right", where), where + "right."),
                   float(_need(d, "left_scale", where)), float(_need(d, "right_scale", where)))

    def to_dict(self):
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class DenseFeedForwardConfig:
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, d, where) -> Optional["DenseFeedForwardConfig"]:
        if d is None:
            return None
        kind = _need(d, "kind", where)
        if kind != "dense":
            raise ConfigError(f"{where}kind={kind!r} is not supported (known: dense)")
        limit = float(_need(d, "limit", where))
        if not limit > 0:
            raise ConfigError(f"{where}limit must be positive, got {limit}")
        return cls(_positive_int(d, "ff", where), limit)

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense", "limit": self.limit}


@dataclass(frozen=True)
class TibepelLayerConfig:
    type: str
    mixer: Union[ScanMixerConfig, ParallelMixerConfig]
    mlp: Optional[DenseFeedForwardConfig]

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


_MIXERS = {"mamba1": ScanMixerConfig, "parallel": ParallelMixerConfig}


@dataclass(frozen=True)
class TibepelConfig:
    vocab: int
    width: int
    layers: Tuple[TibepelLayerConfig, ...]
    embedding_scale: float
    norm_eps: float
    logit_softcap: float
    side_dim: int
    initializer_range: float = 0.02
    eos_token_id: Union[None, int, List[int]] = None

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "TibepelConfig":
        layers = []
        raw_layers = _need(data, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a non-empty list")
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]."
            kind = _need(L, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}type={kind!r} is not supported (known: {sorted(_MIXERS)})")
            layers.append(TibepelLayerConfig(kind, _MIXERS[kind].from_dict(_need(L, "mixer", where), where + "mixer."),
                                             DenseFeedForwardConfig.from_dict(L.get("mlp"), where + "mlp.")))
        width = _positive_int(data, "width", "")
        if width % 2:
            raise ConfigError(f"width={width} must be even: the position vector is made of (sin, cos) pairs")
        eps = float(_need(_need(data, "norm", ""), "eps", "norm."))
        if not eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        eos = data.get("eos_token_id")
        return cls(vocab=_positive_int(data, "vocab", ""), width=width, layers=tuple(layers),
                   embedding_scale=float((data.get("embedding") or {}).get("scale", 1.0)),       # absent: rows as stored
                   norm_eps=eps, logit_softcap=float(data.get("logit_softcap") or 0.0),          # absent or 0: no cap
                   side_dim=_positive_int(_need(data, "token_side", ""), "dim", "token_side."),
                   initializer_range=float(data.get("initializer_range", 0.02)),
                   eos_token_id=[int(e) for e in eos] if isinstance(eos, (list, tuple)) else eos)

    @classmethod
    def from_folder(cls, folder: Union[str, Path]) -> "TibepelConfig":
        return cls.from_dict(json.loads((Path(folder) / "config.json").read_text()))

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": "Tibepel", "embedding": {"scale": self.embedding_scale},
             "layers": [L.to_dict() for L in self.layers], "logit_softcap": self.logit_softcap,
             "norm": {"eps": self.norm_eps}, "token_side": {"dim": self.side_dim}, "vocab": self.vocab, "width": self.width,
             "initializer_range": self.initializer_range}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    @property
    def eos_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        return [self.eos_token_id] if isinstance(self.eos_token_id, int) else list(self.eos_token_id)
