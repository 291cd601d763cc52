"""The Tibepel decoder (architecture name "Tibepel") as a ``ModelSpec``.

The stream starts as embed[token] * scale plus a sinusoidal position vector.  Layer i (tensors
``l<i>.*``) is a pre-norm block: ``norm1`` and a mixer, ``norm2`` and a clamped gated feed-forward
(absent where the layer has none), then a term looked up by the token in the shared table
``side.embed``.  The mixer is a selective scan (type ``mamba1``) or a chunk-masked attention
beside a gated delta rule (type ``parallel``).  Norm weights are stored around zero.  The logits
pass a tanh cap.
"""
from __future__ import annotations

from ..config.tibepel import (ChunkAttentionConfig, DeltaRuleConfig, ParallelMixerConfig, ScanMixerConfig,
                              TibepelConfig)
from ..parts.base import PartSpec, TensorSpec
from .spec import ModelSpec, RunEntry, SharedTensor


def _names(prefix: str, *locals_: str):
    return {n: prefix + n for n in locals_}


def _scan_mixer(width: int, m: ScanMixerConfig, p: str) -> PartSpec:
    return PartSpec("selective_scan", {"hidden": width, "inner": m.inner, "state": m.state, "dt_rank": m.dt_rank, "taps": m.conv},
                    _names(p, "in", "conv", "conv.b", "x", "dt", "dt.b", "A_log", "D", "o"))


def _chunk_attention(width: int, m: ChunkAttentionConfig, p: str, eps: float) -> PartSpec:
    return PartSpec("chunk_attention",
                    {"hidden": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                     "scale": m.scale, "chunk": m.mask_size, "bias": True, "distance_bias": True, "mix_heads": True,
                     "value_norm_eps": eps},
                    _names(p, "q", "q.b", "k", "k.b", "v", "v.b", "r1", "r2", "talk", "o", "o.b"))


def _delta_rule(width: int, m: DeltaRuleConfig, p: str, eps: float) -> PartSpec:
    return PartSpec("gated_delta_rule",
                    {"hidden": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                     "taps": m.conv, "norm_eps": eps, "unit_eps": 1e-6},
                    _names(p, "q", "q.conv", "k", "k.conv", "v", "v.conv", "b", "a", "A_log", "dt_bias", "norm", "g", "o"))


def tibepel_spec(cfg: TibepelConfig, norm_init: str = "zeros") -> ModelSpec:
    """``norm_init``: how random-weights mode draws the norm weights ("zeros", or "zeros_jitter")."""
    W, eps = cfg.width, cfg.norm_eps
    norm = {"width": W, "eps": eps, "offset": 1.0, "init": norm_init}
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        if isinstance(L.mixer, ScanMixerConfig):
            mixer = _scan_mixer(W, L.mixer, p + "mix.")
        else:
            m: ParallelMixerConfig = L.mixer
            mixer = PartSpec("parallel", {"hidden": W, "scales": {"left": m.left_scale, "right": m.right_scale}},
                             parts={"left": _chunk_attention(W, m.left, p + "mix.left.", eps),
                                    "right": _delta_rule(W, m.right, p + "mix.right.", eps)})
        parts = {"norm1": PartSpec("rmsnorm", dict(norm), {"weight": p + "norm1"}), "mixer": mixer,
                 "token_input": PartSpec("gated_side", {"hidden": W, "dim": cfg.side_dim, "column": i * cfg.side_dim,
                                                        "table": "side.embed", "eps": eps},
                                         _names(p + "side.", "gate", "proj", "norm"))}
        if L.mlp is not None:
            parts["norm2"] = PartSpec("rmsnorm", dict(norm), {"weight": p + "norm2"})
            parts["ffn"] = PartSpec("clamped_glu", {"hidden": W, "inter": L.mlp.ff, "limit": L.mlp.limit, "alpha": 1.702,
                                                    "up_shift": 1.0},
                                    _names(p + "mlp.", "gate", "gate.b", "up", "up.b", "down", "down.b"))
        layers.append(PartSpec("pre_norm", parts=parts))
    return ModelSpec(
        architecture="Tibepel", hidden_size=W, vocab_size=cfg.vocab, embedding="embed", layers=layers,
        run_order=[RunEntry(layer=i, cache=i) for i in range(len(layers))],
        final_norm=PartSpec("rmsnorm", dict(norm), {"weight": "final.norm"}), lm_head="head",
        initializer_range=cfg.initializer_range, eos_token_ids=cfg.eos_token_ids,
        embedding_scale=cfg.embedding_scale, position_vector="sinusoidal", position_base=10000.0,
        logit_softcap=cfg.logit_softcap,
        shared_tensors={"side.embed": SharedTensor("side.embed", TensorSpec((cfg.vocab, len(layers) * cfg.side_dim)))})
