"""The Lilenex decoder written out plainly: float64, whole sequences, one function per mechanism.

Shares no code with the package; the package is tested against this.  ``cfg`` is the nested
dictionary of a config.json, ``W`` a dictionary name -> tensor (any element type; promoted here).

Notation: h input of a sub-layer [T, width]; p positions 0..T-1; H query heads, G key/value heads,
d query/key head size, e value head size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w.to(F)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: Optional[dict]):
    """(frequency of pair i [dims/2], factor on cos and sin) of a ``rot`` block; (None, 1) without one."""
    if not rot:
        return None, 1.0
    n, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(n // 2, dtype=F)
    f = base ** (-2.0 * i / n)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_to_dim(turns):
        return n * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_to_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_to_dim(float(sc["slow"]))), n - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, d]: neighbours (2i, 2i+1) of the first ``dims`` entries of every head are turned by p * f_i."""
    f, amp = rotary_frequencies(rot)
    if f is None:
        return x
    n = int(rot["dims"])
    a = positions.to(F)[:, None] * f[None, :]
    c, s = (a.cos() * amp)[:, None, :], (a.sin() * amp)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- attention
def visible(T: int, mask: Optional[dict]) -> torch.Tensor:
    """[T, T] bool: query i sees key j."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if mask and mask.get("size"):
        ok = ok & ((i - j < int(mask["size"])) | (j < int(mask.get("keep_first") or 0)))
    return ok


def attention_keys_values(h, m: dict, W, p: str, eps: float):
    """Keys after norm and rotation [T, G, d] and values [T, G, e] of a layer that has its own."""
    T = h.shape[0]
    G, d, e = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = h @ W[p + "k"].to(F).T
    k = rms_norm(k, W[p + "k.norm"], eps).view(T, G, d)
    k = rotate_pairs(k, torch.arange(T), m.get("rot"))
    v = (h @ W[p + "v"].to(F).T).view(T, G, e)
    return k, v


def attention_mixer(h, m: dict, W, p: str, eps: float, kv):
    """``kv``: (keys, values) of the layer that provides them (this one or an earlier one)."""
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = h @ W[p + "q"].to(F).T
    q = rms_norm(q, W[p + "q.norm"], eps).view(T, H, d)
    q = rotate_pairs(q, torch.arange(T), m.get("rot"))
    k, v = kv
    see = visible(T, m.get("mask"))
    out = torch.zeros(T, H, e, dtype=F)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~see, float("-inf"))
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * e) @ W[p + "o"].to(F).T


# ----------------------------------------------------------------------------- gated linear attention
def gla_mixer(h, m: dict, W, p: str, eps: float, state: Optional[torch.Tensor] = None, return_state: bool = False):
    T = h.shape[0]
    H, d, e, tau = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    q = (h @ W[p + "q"].to(F).T).view(T, H, d) * d ** -0.5
    k = (h @ W[p + "k"].to(F).T).view(T, H, d)
    v = (h @ W[p + "v"].to(F).T).view(T, H, e)
    z = (h @ W[p + "a1"].to(F).T) @ W[p + "a2"].to(F).T + W[p + "a2.b"].to(F)
    decay = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, d)
    S = torch.zeros(H, d, e, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, e, dtype=F)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    o = rms_norm(o, W[p + "norm"], eps).reshape(T, H * e)
    y = (o * silu(h @ W[p + "g"].to(F).T)) @ W[p + "o"].to(F).T
    return (y, S) if return_state else y


# ----------------------------------------------------------------------------- feed-forward
def dense_ff(h, W, p: str):
    return gelu_tanh(h @ W[p + "up"].to(F).T) @ W[p + "down"].to(F).T


def gated_expert(h, W, p: str):
    return (silu(h @ W[p + "gate"].to(F).T) * (h @ W[p + "up"].to(F).T)) @ W[p + "down"].to(F).T


def routed_ff(h, mlp: dict, W, p: str):
    n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    score = torch.sigmoid(h @ W[p + "router"].to(F).T)
    chosen = score.topk(top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for x in chosen[t].tolist():
            out[t] += gated_expert(score[t, x] * h[t:t + 1], W, f"{p}e{x}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, W, p + "shared.")
    return out


def feed_forward(h, mlp: dict, W, p: str):
    if mlp["kind"] == "dense":
        return dense_ff(h, W, p)
    if mlp["kind"] == "moe":
        return routed_ff(h, mlp, W, p)
    raise ValueError(mlp["kind"])


# ----------------------------------------------------------------------------- the model
def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer, summed over its copies)."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    n_streams = int(cfg.get("streams") or 0)
    x0 = W["embed"].to(F)[torch.tensor(tokens, dtype=torch.long)]
    xs = [x0.clone() for _ in range(max(n_streams, 1))]
    kv_of: Dict[int, tuple] = {}
    after = []

    def sublayer(q: int, p: str, fn):
        nonlocal xs
        if n_streams:
            u = sum(float(W[f"{p}hc{q}.in"][s]) * xs[s] for s in range(n_streams))
        else:
            u = xs[0]
        y = fn(rms_norm(u, W[f"{p}norm{q}"], eps))
        if n_streams:
            mix, out = W[f"{p}hc{q}.mix"].to(F), W[f"{p}hc{q}.out"].to(F)
            xs = [sum(mix[s, t] * xs[s] for s in range(n_streams)) + mult * out[t] * y for t in range(n_streams)]
        else:
            xs = [xs[0] + mult * y]

    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        if L["type"] == "attention":
            def mixer(h, m=m, p=p, i=i):
                src = m.get("kv_from")
                if src is None:
                    kv_of[i] = attention_keys_values(h, m, W, p + "mix.", eps)
                    src = i
                return attention_mixer(h, m, W, p + "mix.", eps, kv_of[src])
        elif L["type"] == "gla":
            def mixer(h, m=m, p=p):
                return gla_mixer(h, m, W, p + "mix.", eps)
        else:
            raise ValueError(L["type"])
        sublayer(1, p, mixer)
        if L.get("mlp"):
            sublayer(2, p, lambda h, L=L, p=p: feed_forward(h, L["mlp"], W, p + "mlp."))
        after.append(sum(xs))
    x = rms_norm(sum(xs), W["final.norm"], eps)
    logits = x @ W["embed"].to(F).T
    return (logits, torch.stack(after)) if return_layers else logits


# ----------------------------------------------------------------------------- random models for the tests
def tensor_shapes(cfg: dict, rank: int = 6) -> Dict[str, tuple]:
    """Name -> shape of every tensor of a model (``rank``: inner size of the decay projections)."""
    W, S = int(cfg["width"]), int(cfg.get("streams") or 0)
    out = {"embed": (int(cfg["vocab"]), W), "final.norm": (W,)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (W,)
        subs = [1]
        if L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.q.norm": (H * d,), p + "mix.o": (W, H * e)})
            if m.get("kv_from") is None:
                out.update({p + "mix.k": (G * d, W), p + "mix.v": (G * e, W), p + "mix.k.norm": (G * d,)})
        else:
            H, d, e = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * e, W), p + "mix.g": (H * e, W),
                        p + "mix.o": (W, H * e), p + "mix.norm": (e,), p + "mix.a1": (rank, W), p + "mix.a2": (H * d, rank),
                        p + "mix.a2.b": (H * d,)})
        mlp = L.get("mlp")
        if mlp:
            subs.append(2)
            out[p + "norm2"] = (W,)
            if mlp["kind"] == "dense":
                out.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                ff = mlp["expert"]["ff"]
                out[p + "mlp.router"] = (mlp["router"]["experts"], W)
                for x in range(mlp["router"]["experts"]):
                    out.update({f"{p}mlp.e{x}.gate": (ff, W), f"{p}mlp.e{x}.up": (ff, W), f"{p}mlp.e{x}.down": (W, ff)})
                if mlp.get("shared"):
                    sf = mlp["shared"]["ff"]
                    out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
        for q in subs if S else []:
            out.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
    return out


def random_weights(cfg: dict, seed: int, dtype=torch.float32, rank: int = 6) -> Dict[str, torch.Tensor]:
    """Weights drawn so that no mechanism drowns: matrices N(0, 1.5^2 / fan_in), decays near one, copies of the
    stream that mix but do not blow up, router logits that spread."""
    gen = torch.Generator().manual_seed(seed)
    rand = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
    uni = lambda lo, hi, *s: lo + (hi - lo) * torch.rand(*s, generator=gen, dtype=torch.float32)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg, rank).items()):
        last = name.split(".")[-1]
        if name == "embed":
            t = rand(*shape) * 0.7
        elif last in ("norm1", "norm2", "norm") or name == "final.norm":
            t = 1 + 0.2 * rand(*shape)
        elif last == "in":
            t = uni(0.2, 0.8, *shape)
        elif last == "out":
            t = uni(0.4, 1.0, *shape)
        elif last == "mix":
            t = torch.eye(shape[0]) * 0.6 + 0.3 * uni(0, 1, *shape)
        elif last == "b":
            t = uni(0.5, 4.0, *shape)
        elif last == "router":
            t = rand(*shape) * (3.0 / math.sqrt(shape[-1]))
        else:
            t = rand(*shape) * (1.5 / math.sqrt(shape[-1]))
        out[name] = t.to(dtype)
    return out


def write_model(folder, cfg: dict, seed: int, dtype=torch.float32, weights=None):
    """A model folder (config.json, model.safetensors); returns the weights as stored."""
    import json
    from pathlib import Path
    from pytriton_llama_b200.weights import write_file      # only the file format comes from the package
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    W = weights if weights is not None else random_weights(cfg, seed, dtype)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_file(folder / "model.safetensors", W)
    return W


def attention(heads, kv_heads, dim, vdim, scale, size=0, keep_first=0, rot=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size, "keep_first": keep_first}
    if rot:
        m["rot"] = rot
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def rotation(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def gla(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(vocab, width, layers, streams=0, mult=1.0, eps=1e-5):
    c = {"architecture": "Lilenex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if streams:
        c["streams"] = streams
    return c


_ROT_A = rotation(8, 1000.0, (4.0, 32, 8.0, 1.0))
# Two copies of the stream; value heads larger than key heads; a layer that reads another's keys through a wider
# window with more kept positions; two experts per token; a layer without a feed-forward that sees everything and
# rotates whole heads without scaling; windows that straddle pages of 4, 8 and 16.
TINY_A = config(97, 48, [
    layer("attention", attention(4, 2, 16, 24, 0.3, size=11, keep_first=3, rot=_ROT_A), dense(40)),
    layer("gla", gla(3, 8, 12, 4.0), moe(24, 5, 2, shared=16)),
    layer("attention", attention(4, 2, 16, 24, 0.25, size=19, keep_first=5, rot=_ROT_A, kv_from=0), moe(16, 4, 1)),
    layer("attention", attention(2, 1, 24, 16, 0.2, rot=rotation(24, 300.0)), None),
], streams=2, mult=0.7)
# One stream with a plain residual sum; a single linear-attention head wider than a warp's packet; as many kv heads as
# heads, no rotation, no kept positions; every expert chosen; a layer without a feed-forward.
TINY_B = config(70, 64, [
    layer("gla", gla(1, 20, 40, 16.0), dense(72)),
    layer("attention", attention(6, 6, 16, 16, 0.35, size=7), moe(24, 3, 3, shared=24)),
    layer("gla", gla(2, 32, 8, 2.0), None),
], eps=3e-4)
# Four copies; one kv head for three query heads; more kept positions than the window is wide; a reader whose window
# is narrower than its source's.
TINY_C = config(50, 32, [
    layer("attention", attention(3, 1, 16, 32, 0.3, size=8, keep_first=9, rot=rotation(16, 50.0, (2.0, 16, 4.0, 0.5))), moe(16, 6, 2)),
    layer("attention", attention(3, 1, 16, 32, 0.3, size=5, keep_first=2, rot=rotation(16, 50.0, (2.0, 16, 4.0, 0.5)), kv_from=0), dense(48)),
], streams=4, mult=0.4)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
