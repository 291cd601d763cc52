"""Gated linear attention: a matrix state per head that decays per key channel.

With h the mixer's input: q = W_q h * head_dim^(-1/2), k = W_k h (heads x head_dim), v = W_v h (heads x
value_dim); the decay of key channel c is a = sigmoid(z_c)^(1/tau) with z = W_a2 (W_a1 h) + b.  Per head

    S <- diag(a) S + k v^T        o = S^T q

o is divided by its root mean square per head and multiplied by ``norm`` [value_dim]; the heads are
concatenated, multiplied by silu(W_g h) and projected by W_o.  S [heads, head_dim, value_dim] is
per-request state: float32, zero before position 0.  The projections run in the compute type; z,
the decay (kept as its logarithm), the state and the read-out are float32.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Part):
    """params: ``hidden``, ``heads``, ``head_dim``, ``value_dim``, ``tau``, ``norm_eps``, ``decay_rank`` (the inner size
    of the decay projection when weights are drawn at random; a checkpoint's own size is taken as it is).
    Tensors: ``q``, ``k`` [heads*head_dim, hidden], ``v``, ``g`` [heads*value_dim, hidden], ``a1`` [rank, hidden],
    ``a2`` [heads*head_dim, rank], ``a2.b`` [heads*head_dim], ``norm`` [value_dim], ``o`` [hidden, heads*value_dim]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.d, self.dv = int(p["head_dim"]), int(p["value_dim"])
        self.tau, self.norm_eps = float(p["tau"]), float(p["norm_eps"])
        self.rank = int(p.get("decay_rank") or 16)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H, d, dv, W = self.heads, self.d, self.dv, self.hidden
        return {"q": TensorSpec((H * d, W)), "k": TensorSpec((H * d, W)), "v": TensorSpec((H * dv, W)), "g": TensorSpec((H * dv, W)),
                "a1": TensorSpec((-self.rank, W)), "a2": TensorSpec((H * d, -self.rank)),
                "a2.b": TensorSpec((H * d,), "uniform", lo=1.0, hi=5.0), "norm": TensorSpec((dv,), "ones"),
                "o": TensorSpec((W, H * dv))}

    def load(self, t) -> None:
        if t["a1"].shape[0] != t["a2"].shape[1]:
            raise ValueError(f"the decay projections do not fit: a1 is {list(t['a1'].shape)}, a2 is {list(t['a2'].shape)}")
        self.w_qkvg = self._to_compute(torch.cat([t["q"], t["k"], t["v"], t["g"]], dim=0))
        self.w_a1 = self._to_compute(t["a1"])
        self.w_a2 = self._to_f32(t["a2"])           # the second, small product runs in float32 on the float32 result of the first
        self.a_bias, self.norm_w = self._to_f32(t["a2.b"]), self._to_f32(t["norm"])
        self.w_o = self._to_compute(t["o"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", states=(("S", (self.heads, self.d, self.dv)),))

    def forward(self, x, ctx, cache):
        ops = self.rt.ops
        H, d, dv = self.heads, self.d, self.dv
        proj = ops.linear(x, self.w_qkvg)                                     # [T, q | k | v | gate]
        z = ops.linear_simt(ops.linear(x, self.w_a1, out_dtype=torch.float32), self.w_a2)     # float32 [T, heads*head_dim], before the bias
        o = ops.gla_scan(proj, z, self.a_bias, 1.0 / self.tau, cache.states["S"], ctx, H, d, dv, d ** -0.5)
        out = ops.empty((proj.shape[0], H * dv), self.rt.dtype)
        ops.gated_head_norm(o, self.norm_w, self.norm_eps, proj, 2 * H * d + H * dv, H, dv, out, 0, 1.0)
        return ops.linear(out, self.w_o)
