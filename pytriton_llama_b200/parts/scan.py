"""Selective scan (the recurrent mixer of Mamba's first form).

With h the mixer's input:  [x | z] = W_in h;  x <- silu(conv(x)) (causal, per channel, with bias);
[dt | B | C] = W_x x;  dt <- softplus(W_dt dt + b_dt);  A = -exp(A_log).  Per channel c and state n

    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n        y_c = sum_n S[c, n] C_n + D_c x_c

and the output is W_o (y * silu(z)).  S and the last ``taps - 1`` inputs of the convolution are
per-request state (float32, zero before position 0).  Projections and the convolution run in the
compute type; step sizes, decays and the state are float32.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("mixer", "selective_scan")
class SelectiveScan(Part):
    """params: ``hidden``, ``inner``, ``state``, ``dt_rank``, ``taps``.  Tensors: ``in`` [2*inner, hidden],
    ``conv`` [inner, taps], ``conv.b`` [inner], ``x`` [dt_rank + 2*state, inner], ``dt`` [inner, dt_rank],
    ``dt.b`` [inner], ``A_log`` [inner, state], ``D`` [inner], ``o`` [hidden, inner]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.inner, self.state = int(p["hidden"]), int(p["inner"]), int(p["state"])
        self.dt_rank, self.taps = int(p["dt_rank"]), int(p["taps"])

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        i, n, r = self.inner, self.state, self.dt_rank
        return {"in": TensorSpec((2 * i, self.hidden)), "conv": TensorSpec((i, self.taps), "uniform", lo=-0.5, hi=0.5),
                "conv.b": TensorSpec((i,), "zeros_jitter"), "x": TensorSpec((r + 2 * n, i)), "dt": TensorSpec((i, r)),
                "dt.b": TensorSpec((i,), "uniform", lo=-4.0, hi=-1.0), "A_log": TensorSpec((i, n), "uniform", lo=-1.0, hi=2.0),
                "D": TensorSpec((i,), "ones"), "o": TensorSpec((self.hidden, i))}

    def load(self, t) -> None:
        self.w_in = self._to_compute(t["in"])
        self.conv_w, self.conv_b = self._to_f32(t["conv"]), self._to_f32(t["conv.b"])
        self.w_x_dt = self._to_compute(t["x"][:self.dt_rank])          # two products, so that each result is contiguous
        self.w_x_bc = self._to_compute(t["x"][self.dt_rank:])
        self.w_dt, self.dt_b = self._to_compute(t["dt"]), self._to_f32(t["dt.b"])
        self.A = -torch.exp(self._to_f32(t["A_log"]))
        self.D = self._to_f32(t["D"])
        self.w_o = self._to_compute(t["o"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="none", states=(("conv", (max(self.taps - 1, 1), self.inner)), ("scan", (self.inner, self.state))))

    def forward(self, x, ctx, cache):
        ops = self.rt.ops
        xz = ops.linear(x, self.w_in)
        xc = ops.causal_conv(xz, 0, self.inner, self.conv_w, self.conv_b, cache.states["conv"], ctx, silu=True)
        dt = ops.linear(ops.linear(xc, self.w_x_dt), self.w_dt, out_dtype=torch.float32)
        bc = ops.linear(xc, self.w_x_bc)
        y = ops.selective_scan(xc, dt, self.dt_b, self.A, bc, self.D, xz, self.inner, cache.states["scan"], ctx)
        return ops.linear(y, self.w_o)
