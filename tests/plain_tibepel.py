"""A plain, slow statement of the Tibepel decoder in float64 on the CPU: one function per mechanism,
whole sequences only, recurrences walked token by token.  It shares nothing with the package: it
reads config.json's keys and the checkpoint's tensor names itself.  Also makes random models whose
weights are scaled so that every mechanism matters in the logits.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

F = torch.float64


# ---------------------------------------------------------------------------- small functions
def rms_div(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    return rms_div(x, eps) * (1 + w)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def causal_conv(x, w, b=None):
    """x [T, C]; w [C, taps], last column the current token's; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for k in range(taps):
        y = y + padded[k:k + T] * w[:, k]
    return y if b is None else y + b


def position_vector(T, width, base=10000.0):
    pos = torch.arange(T, dtype=F)[:, None]
    i = torch.arange(width // 2, dtype=F)[None, :]
    ang = pos * base ** (-2 * i / width)
    pe = torch.zeros(T, width, dtype=F)
    pe[:, 0::2] = torch.sin(ang)
    pe[:, 1::2] = torch.cos(ang)
    return pe


# ---------------------------------------------------------------------------- mechanisms
def selective_scan_mixer(h, W, p, m):
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    proj = x @ W[p + "x"].T
    dt, B, C = proj[:, :R], proj[:, R:R + N], proj[:, R + N:]
    dt = softplus(dt @ W[p + "dt"].T + W[p + "dt.b"])
    A = -torch.exp(W[p + "A_log"])
    S = torch.zeros(inner, N, dtype=F)
    ys = []
    for t in range(h.shape[0]):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        ys.append(S @ C[t] + W[p + "D"] * x[t])
    return (torch.stack(ys) * silu(z)) @ W[p + "o"].T


def attention_weights(q, k, m, r1, r2):
    """softmax weights [H, T, T] of the chunk-masked attention with the distance bias."""
    H, G, size = m["heads"], m["kv_heads"], m["mask"]["size"]
    T = q.shape[0]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = (j <= i) & ((i // size) == (j // size))
    dist = (i - j).clamp(min=0).to(F)
    P = torch.zeros(H, T, T, dtype=F)
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * m["scale"] - r1[h] * torch.log1p(r2[h] * dist)
        P[h] = torch.softmax(s.masked_fill(~visible, float("-inf")), -1)
    return P


def chunk_attention_mixer(h, W, p, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, d)
    v = rms_div((h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, dv), eps)
    P = torch.einsum("hg,gij->hij", W[p + "talk"], attention_weights(q, k, m, W[p + "r1"], W[p + "r2"]))
    o = torch.stack([P[hh] @ v[:, hh // (H // G)] for hh in range(H)], 1).reshape(T, H * dv)
    return o @ W[p + "o"].T + W[p + "o.b"]


def delta_rule_mixer(h, W, p, m, eps):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    S = torch.zeros(H, d, dv, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        for hh in range(H):
            c = hh // (H // G)
            S[hh] = g[t, hh] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ k[t, c])
            S[hh] = S[hh] + torch.outer(k[t, c], u)
            out[t, hh] = S[hh].T @ q[t, c]
    out = (rms_div(out, eps) * W[p + "norm"]).reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


def clamped_feed_forward(h, W, p, m):
    limit = m["limit"]
    g = torch.clamp(h @ W[p + "gate"].T + W[p + "gate.b"], max=limit)
    u = torch.clamp(h @ W[p + "up"].T + W[p + "up.b"], -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[p + "down"].T + W[p + "down.b"]


def side_term(x, tok, W, p, layer, dim, eps):
    e = W["side.embed"][tok][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ W[p + "gate"].T) * e) @ W[p + "proj"].T
    return rms_div(y, eps) * W[p + "norm"]


# ---------------------------------------------------------------------------- the model
def forward(cfg, W, tokens, streams=None):
    """float64 logits [T, vocab] of a whole sequence; ``streams`` (a list) receives the stream after every layer."""
    W = {k: v.to(F) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.tensor(tokens)
    x = W["embed"][tok] * cfg["embedding"]["scale"] + position_vector(len(tokens), cfg["width"])
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        h = norm_around_zero(x, W[p + "norm1"], eps)
        if L["type"] == "mamba1":
            x = x + selective_scan_mixer(h, W, p + "mix.", L["mixer"])
        else:
            m = L["mixer"]
            x = x + m["left_scale"] * chunk_attention_mixer(h, W, p + "mix.left.", m["left"], eps) \
                  + m["right_scale"] * delta_rule_mixer(h, W, p + "mix.right.", m["right"], eps)
        if L["mlp"] is not None:
            x = x + clamped_feed_forward(norm_around_zero(x, W[p + "norm2"], eps), W, p + "mlp.", L["mlp"])
        x = x + side_term(x, tok, W, p + "side.", li, cfg["token_side"]["dim"], eps)
        if streams is not None:
            streams.append(x.clone())
    logits = norm_around_zero(x, W["final.norm"], eps) @ W["head"].T
    cap = cfg["logit_softcap"]
    return cap * torch.tanh(logits / cap)


# ---------------------------------------------------------------------------- random models
def tensor_shapes(cfg):
    Wd, V = cfg["width"], cfg["vocab"]
    sd = cfg["token_side"]["dim"]
    out = {"embed": (V, Wd), "side.embed": (V, len(cfg["layers"]) * sd), "final.norm": (Wd,), "head": (V, Wd)}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        out[p + "norm1"] = (Wd,)
        m = L["mixer"]
        if L["type"] == "mamba1":
            I, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
            out.update({p + "mix.in": (2 * I, Wd), p + "mix.conv": (I, K), p + "mix.conv.b": (I,), p + "mix.x": (R + 2 * N, I),
                        p + "mix.dt": (I, R), p + "mix.dt.b": (I,), p + "mix.A_log": (I, N), p + "mix.D": (I,), p + "mix.o": (Wd, I)})
        else:
            a, b = m["left"], m["right"]
            q = p + "mix.left."
            out.update({q + "q": (a["heads"] * a["dim"], Wd), q + "q.b": (a["heads"] * a["dim"],),
                        q + "k": (a["kv_heads"] * a["dim"], Wd), q + "k.b": (a["kv_heads"] * a["dim"],),
                        q + "v": (a["kv_heads"] * a["vdim"], Wd), q + "v.b": (a["kv_heads"] * a["vdim"],),
                        q + "r1": (a["heads"],), q + "r2": (a["heads"],), q + "talk": (a["heads"], a["heads"]),
                        q + "o": (Wd, a["heads"] * a["vdim"]), q + "o.b": (Wd,)})
            q = p + "mix.right."
            cq, cv = b["kv_heads"] * b["dim"], b["heads"] * b["vdim"]
            out.update({q + "q": (cq, Wd), q + "q.conv": (cq, b["conv"]), q + "k": (cq, Wd), q + "k.conv": (cq, b["conv"]),
                        q + "v": (cv, Wd), q + "v.conv": (cv, b["conv"]), q + "b": (b["heads"], Wd), q + "a": (b["heads"], Wd),
                        q + "A_log": (b["heads"],), q + "dt_bias": (b["heads"],), q + "norm": (b["vdim"],), q + "g": (cv, Wd),
                        q + "o": (Wd, cv)})
        if L["mlp"] is not None:
            ff = L["mlp"]["ff"]
            out.update({p + "norm2": (Wd,), p + "mlp.gate": (ff, Wd), p + "mlp.gate.b": (ff,), p + "mlp.up": (ff, Wd),
                        p + "mlp.up.b": (ff,), p + "mlp.down": (Wd, ff), p + "mlp.down.b": (Wd,)})
        out.update({p + "side.gate": (sd, Wd), p + "side.proj": (Wd, sd), p + "side.norm": (Wd,)})
    return out


def random_weights(cfg, seed, dtype=torch.float32):
    """Weights drawn so that no mechanism drowns: matrices N(0, 1/fan_in), small biases, decays spread out."""
    gen = torch.Generator().manual_seed(seed)
    rand = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
    uni = lambda lo, hi, *s: lo + (hi - lo) * torch.rand(*s, generator=gen, dtype=torch.float32)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        last = name.split(".")[-1]
        if name in ("embed", "side.embed"):
            t = rand(*shape) * (0.5 if name == "embed" else 1.0)
        elif last in ("norm1", "norm2") or name == "final.norm":
            t = 0.2 * rand(*shape)
        elif name.endswith("side.norm") or name.endswith("right.norm"):
            t = 1 + 0.2 * rand(*shape)
        elif last == "conv":
            t = uni(-0.6, 0.6, *shape)
        elif last == "b" and len(shape) == 1:
            t = 0.3 * rand(*shape) if not name.endswith("dt.b") else uni(-3.0, -0.5, *shape)
        elif last == "A_log":
            t = uni(-1.0, 1.5, *shape)
        elif last == "dt_bias":
            t = uni(-2.0, 1.0, *shape)
        elif last == "D":
            t = 1 + 0.3 * rand(*shape)
        elif last == "r1":
            t = uni(0.0, 1.5, *shape)
        elif last == "r2":
            t = uni(0.05, 2.0, *shape)
        elif last == "talk":
            t = torch.eye(shape[0]) * 0.7 + 0.3 * rand(*shape)
        else:
            t = rand(*shape) * (1.5 / math.sqrt(shape[-1]))
        out[name] = t.to(dtype)
    return out


def write_model(folder, cfg, seed, dtype=torch.float32):
    """A model folder (config.json, model.safetensors) of random weights; returns the weights as stored."""
    from pytriton_llama_b200.weights import write_file      # only the file format comes from the package
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    W = random_weights(cfg, seed, dtype)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_file(folder / "model.safetensors", W)
    return W


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def scan(inner, state, dt_rank, conv):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def parallel(left, right, left_scale, right_scale):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def left(heads, kv_heads, dim, vdim, size, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size}, "scale": scale}


def right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(vocab, width, side, layers, scale=3.0, eps=1e-5, cap=20.0):
    return {"architecture": "Tibepel", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "logit_softcap": cap, "token_side": {"dim": side}, "layers": layers}


# Sizes that are not multiples of anything convenient; value heads of another size than key heads; as many kv heads as
# heads on the left and fewer on the right; a layer without a feed-forward; blocks of 8 positions against pages of 4 or 16.
TINY_P = config(96, 64, 8, [
    layer("parallel", parallel(left(4, 4, 16, 24, 8, 0.3), right(4, 2, 8, 16, 3), 0.7, 1.3), dense(72, 1.5)),
    layer("mamba1", scan(48, 5, 3, 2), None),
    layer("parallel", parallel(left(2, 1, 24, 8, 8, 0.2), right(2, 2, 20, 12, 2), 1.0, 0.4), dense(40, 3.0)),
])
# one head on the right, a block of 24 positions (pages of 16 straddle it), many taps, a state that needs several lanes' turns
TINY_Q = config(130, 96, 4, [
    layer("mamba1", scan(80, 20, 6, 5), dense(112, 2.5)),
    layer("parallel", parallel(left(6, 2, 32, 16, 24, 0.18), right(1, 1, 40, 24, 4), 0.5, 0.9), None),
    layer("mamba1", scan(36, 9, 2, 3), dense(64, 1.0)),
], scale=2.0, eps=3e-4, cap=12.0)
TINY = {"P": TINY_P, "Q": TINY_Q}
