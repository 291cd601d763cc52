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
