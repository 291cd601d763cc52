"""Gated feed-forward with clamped branches: g = min(W_gate h + b, limit), u = clamp(W_up h + b,
-limit, limit), y = g * sigmoid(alpha * g) * (u + up_shift), output W_down y (+ bias, left for the
caller: ``output_bias``).  Gate and up are one [2*inter, hidden] weight, gate rows first."""
from __future__ import annotations

from typing import Dict

import torch

from .base import Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("ffn", "clamped_glu")
class ClampedGLU(Part):
    """params: ``hidden``, ``inter``, ``limit``, ``alpha``, ``up_shift``.  Tensors: ``gate``, ``up`` [inter, hidden],
    ``down`` [hidden, inter] and their biases ``gate.b``, ``up.b``, ``down.b``."""

    output_bias_spec = True

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.inter = int(p["hidden"]), int(p["inter"])
        self.limit, self.alpha, self.up_shift = float(p["limit"]), float(p.get("alpha", 1.702)), float(p.get("up_shift", 1.0))
        self.output_bias = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"gate": TensorSpec((self.inter, self.hidden)), "up": TensorSpec((self.inter, self.hidden)),
                "down": TensorSpec((self.hidden, self.inter)), "gate.b": TensorSpec((self.inter,), "zeros_jitter"),
                "up.b": TensorSpec((self.inter,), "zeros_jitter"), "down.b": TensorSpec((self.hidden,), "zeros_jitter")}

    def load(self, t) -> None:
        self.w_gate_up = self._to_compute(torch.cat([t["gate"], t["up"]], dim=0))
        self.b_gate_up = self._to_f32(torch.cat([t["gate.b"], t["up.b"]], dim=0))
        self.w_down = self._to_compute(t["down"])
        self.output_bias = self._to_f32(t["down.b"])

    def forward(self, x):
        ops = self.rt.ops
        y = ops.clamped_glu(ops.linear(x, self.w_gate_up), self.b_gate_up, self.limit, self.alpha, self.up_shift)
        return ops.linear(y, self.w_down)
