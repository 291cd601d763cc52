"""The Lilenex decoder (architecture name "Lilenex") as a ``ModelSpec``.

Layer i (tensors ``l<i>.*``) is a pre-norm block over ``streams`` copies of the residual stream
(``hc1.*`` around the mixer, ``hc2.*`` around the feed-forward; without copies a plain residual sum
with the multiplier ``residual_mult``).  The mixer is a windowed softmax attention that keeps the
first positions (``attention``; with ``kv_from`` it reads the cache entry of an earlier layer) or
gated linear attention (``gla``); the feed-forward is a gelu layer, a routed mixture of gated
experts with a shared one, or absent.  The logits come from the embedding table.
"""
from __future__ import annotations

from ..config.lilenex import AttentionMixerConfig, DenseMlpConfig, GlaMixerConfig, LilenexConfig, MoeMlpConfig
from ..parts.base import PartSpec
from .spec import ModelSpec, RunEntry


def _names(prefix: str, *locals_: str):
    return {n: prefix + n for n in locals_}


def _attention(width: int, m: AttentionMixerConfig, p: str, eps: float) -> PartSpec:
    own = m.kv_from is None
    names = ["q", "q.norm", "o"] + (["k", "v", "k.norm"] if own else [])
    parts = {}
    if m.rot is not None:
        sc = m.rot.scaling
        parts["position"] = PartSpec("rotary_pairs", {"head_dim": m.dim, "dims": m.rot.dims, "base": m.rot.base,
                                                      "scaling": None if sc is None else sc.to_dict()})
    return PartSpec("window_attention",
                    {"hidden": width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                     "scale": m.scale, "window": m.window, "keep_first": m.keep_first, "qk_norm_eps": eps, "own_kv": own},
                    _names(p, *names), parts)


def _gla(width: int, m: GlaMixerConfig, p: str, eps: float) -> PartSpec:
    return PartSpec("gated_linear_attention",
                    {"hidden": width, "heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "tau": m.tau, "norm_eps": eps,
                     "decay_rank": m.rank},
                    _names(p, "q", "k", "v", "g", "a1", "a2", "a2.b", "norm", "o"))


def _feed_forward(width: int, mlp, p: str) -> PartSpec:
    if isinstance(mlp, DenseMlpConfig):
        return PartSpec("gelu_mlp", {"hidden": width, "inter": mlp.ff}, _names(p, "up", "down"))
    m: MoeMlpConfig = mlp
    names = ["router"] + [f"e{i}.{w}" for i in range(m.experts) for w in ("gate", "up", "down")]
    if m.shared_ff:
        names += ["shared.gate", "shared.up", "shared.down"]
    return PartSpec("routed_experts", {"hidden": width, "inter": m.ff, "experts": m.experts, "top": m.top,
                                       "shared_inter": m.shared_ff, "scale_input": True}, _names(p, *names))


def lilenex_spec(cfg: LilenexConfig, norm_init: str = "ones") -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    learned = cfg.streams > 0
    S = max(cfg.streams, 1)

    def norm(weight: str, read=None):
        tensors = {"weight": weight}
        if read is not None:
            tensors["read"] = read
        return PartSpec("stream_rmsnorm", {"width": W, "eps": eps, "streams": S, "learned": read is not None, "init": norm_init}, tensors)

    layers, run_order = [], []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        cache, write = i, True
        if isinstance(L.mixer, AttentionMixerConfig):
            mixer = _attention(W, L.mixer, p + "mix.", eps)
            if L.mixer.kv_from is not None:
                cache, write = L.mixer.kv_from, False
        else:
            mixer = _gla(W, L.mixer, p + "mix.", eps)
        parts = {"norm1": norm(p + "norm1", p + "hc1.in" if learned else None), "mixer": mixer}
        tensors = {"mix1": p + "hc1.mix", "out1": p + "hc1.out"} if learned else {}
        if L.mlp is not None:
            parts["norm2"] = norm(p + "norm2", p + "hc2.in" if learned else None)
            parts["ffn"] = _feed_forward(W, L.mlp, p + "mlp.")
            if learned:
                tensors.update({"mix2": p + "hc2.mix", "out2": p + "hc2.out"})
        layers.append(PartSpec("hyper_connections", {"streams": S, "mult": cfg.residual_mult, "learned": learned}, tensors, parts))
        run_order.append(RunEntry(layer=i, cache=cache, write=write))
    return ModelSpec(architecture="Lilenex", hidden_size=W, vocab_size=cfg.vocab, embedding="embed", layers=layers,
                     run_order=run_order, final_norm=norm("final.norm"), lm_head=None,
                     initializer_range=cfg.initializer_range, eos_token_ids=cfg.eos_token_ids)
