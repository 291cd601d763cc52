"""Gated delta rule: a linear-attention mixer whose state is corrected towards each new value.

q, k = W h (``kv_heads`` heads of ``head_dim``), v = W h (``heads`` heads of ``value_dim``); each
passes a short causal convolution per channel and silu; q and k are scaled to unit length per head
(x / sqrt(sum x^2 + unit_eps)) and q by head_dim^(-1/2).  Per value head (q/k head h // (heads /
kv_heads)), with beta = sigmoid(W_b h) and g = exp(-exp(A_log) * softplus(W_a h + dt_bias)):

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

o is divided by its root mean square per head, multiplied by ``norm`` [value_dim] and by
silu(W_g h), then projected by W_o.  S [heads, head_dim, value_dim] and the last ``taps - 1``
inputs of the convolutions are per-request state (float32, zero before position 0).
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("mixer", "gated_delta_rule")
class GatedDeltaRule(Part):
    """params: ``hidden``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``taps``, ``norm_eps``, ``unit_eps``.
    Tensors: ``q``, ``k`` [kv_heads*head_dim, hidden], ``v``, ``g`` [heads*value_dim, hidden], ``q.conv``, ``k.conv``,
    ``v.conv`` [channels, taps], ``b``, ``a`` [heads, hidden], ``A_log``, ``dt_bias`` [heads], ``norm`` [value_dim],
    ``o`` [hidden, heads*value_dim]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.d, self.dv, self.taps = int(p["head_dim"]), int(p["value_dim"]), int(p["taps"])
        self.norm_eps, self.unit_eps = float(p["norm_eps"]), float(p.get("unit_eps", 1e-6))
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} value heads are no multiple of {self.kv_heads} query/key heads")
        self.conv_channels = 2 * self.kv_heads * self.d + self.heads * self.dv
        self.inner_width = self.heads * self.dv
        self.output_bias = None
        self.w_o = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H, G, d, dv, W = self.heads, self.kv_heads, self.d, self.dv, self.hidden
        conv = lambda c: TensorSpec((c, self.taps), "uniform", lo=-0.5, hi=0.5)
        return {"q": TensorSpec((G * d, W)), "k": TensorSpec((G * d, W)), "v": TensorSpec((H * dv, W)), "g": TensorSpec((H * dv, W)),
                "q.conv": conv(G * d), "k.conv": conv(G * d), "v.conv": conv(H * dv), "b": TensorSpec((H, W)), "a": TensorSpec((H, W)),
                "A_log": TensorSpec((H,), "uniform", lo=-2.0, hi=1.0), "dt_bias": TensorSpec((H,), "uniform", lo=-2.0, hi=1.0),
                "norm": TensorSpec((dv,), "ones"), "o": TensorSpec((W, H * dv))}

    def load(self, t) -> None:
        self.w_qkvg = self._to_compute(torch.cat([t["q"], t["k"], t["v"], t["g"]], dim=0))
        self.conv_w = self._to_f32(torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0))
        self.w_ba = self._to_compute(torch.cat([t["b"], t["a"]], dim=0))
        self.decay_rate = torch.exp(self._to_f32(t["A_log"]))
        self.dt_bias, self.norm_w = self._to_f32(t["dt_bias"]), self._to_f32(t["norm"])
        self.w_o = self._to_compute(t["o"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", states=(("conv", (max(self.taps - 1, 1), self.conv_channels)),
                                              ("S", (self.heads, self.d, self.dv))))

    def write_inner(self, x, ctx, cache, out, column: int, scale: float) -> None:
        ops = self.rt.ops
        proj = ops.linear(x, self.w_qkvg)                                   # [T, q | k | v | gate]
        ba = ops.linear(x, self.w_ba, out_dtype=torch.float32)              # [T, beta's | decay's] before their functions
        qkv = ops.causal_conv(proj, 0, self.conv_channels, self.conv_w, None, cache.states["conv"], ctx, silu=True)
        o = ops.gated_delta_rule(qkv, ba, self.decay_rate, self.dt_bias, cache.states["S"], ctx, self.heads, self.kv_heads,
                                 self.d, self.dv, self.unit_eps, self.d ** -0.5)
        ops.gated_head_norm(o, self.norm_w, self.norm_eps, proj, self.conv_channels, self.heads, self.dv, out, column, scale)

    def forward(self, x, ctx, cache):
        out = self.rt.ops.empty((x.shape[0], self.inner_width), self.rt.dtype)
        self.write_inner(x, ctx, cache, out, 0, 1.0)
        return self.rt.ops.linear(out, self.w_o)
