"""A term of the stream that is looked up by the token itself.

With x the stream after the layer's last sub-layer and e = table[token, column : column + dim]:
g = gelu_tanh(W_gate x) * e;  y = W_proj g;  x <- x + y / sqrt(mean(y^2) + eps) * norm.
The table [vocab, layers * dim] is shared by the layers (``Runtime.shared``); everything here is
float32 arithmetic on the float32 stream.
"""
from __future__ import annotations

from typing import Dict

from .base import Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("token_input", "gated_side")
class GatedSideInput(Part):
    """params: ``hidden``, ``dim``, ``column`` (first column of this layer in the table), ``table`` (key of the
    shared tensor), ``eps``.  Tensors: ``gate`` [dim, hidden], ``proj`` [hidden, dim], ``norm`` [hidden]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.dim, self.column = int(p["hidden"]), int(p["dim"]), int(p["column"])
        self.table_key, self.eps = str(p["table"]), float(p["eps"])

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"gate": TensorSpec((self.dim, self.hidden)), "proj": TensorSpec((self.hidden, self.dim)),
                "norm": TensorSpec((self.hidden,), "ones")}

    def load(self, t) -> None:
        self.w_gate, self.w_proj = self._to_compute(t["gate"]), self._to_compute(t["proj"])
        self.norm_w = self._to_f32(t["norm"])

    def apply(self, residual, x, bias, ctx) -> None:
        self.rt.ops.token_side(residual, x, bias, ctx.tokens, self.rt.shared[self.table_key], self.column, self.dim,
                               self.w_gate, self.w_proj, self.norm_w, self.eps)
