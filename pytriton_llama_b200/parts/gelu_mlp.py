"""Dense feed-forward with one hidden layer: W_down act(W_up h), act the tanh form of gelu,
gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), worked out in float32."""
from __future__ import annotations

from typing import Dict

from .base import Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("ffn", "gelu_mlp")
class GeluMLP(Part):
    """params: ``hidden``, ``inter``.  Tensors: ``up`` [inter, hidden], ``down`` [hidden, inter]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.hidden, self.inter = int(spec.params["hidden"]), int(spec.params["inter"])

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"up": TensorSpec((self.inter, self.hidden)), "down": TensorSpec((self.hidden, self.inter))}

    def load(self, t) -> None:
        self.w_up, self.w_down = self._to_compute(t["up"]), self._to_compute(t["down"])

    def forward(self, x):
        ops = self.rt.ops
        return ops.linear(ops.gelu_tanh(ops.linear(x, self.w_up)), self.w_down)
