"""Grouped-query attention inside blocks of positions, over the paged cache.

q, k, v = W h (+ biases), no rotation.  Each value head is divided by its root mean square
before it is stored (``value_norm_eps`` > 0).  Query i sees key j <= i of the same block of
``chunk`` positions, blocks counted from position 0 of the request (``chunk`` 0: every j <= i):

    score_h(i, j) = (q_h(i) . k(j)) * scale - r1_h * ln(1 + r2_h * (i - j))      (``distance_bias``)
    w_h = softmax_j(score_h);     w'_h = sum_g talk[h, g] w_g                      (``mix_heads``)
    o_h(i) = sum_j w'_h(i, j) v(j)        with k, v of kv head h // (heads / kv_heads)

and the output is W_o o (+ bias, left for the caller: ``output_bias``).  Scores and weights are
float32.  Pages that lie wholly before the block of the next query are given back.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("mixer", "chunk_attention")
class ChunkAttention(Part):
    """params: ``hidden``, ``heads``, ``kv_heads``, ``head_dim``, ``value_dim``, ``scale``, ``chunk``; flags ``bias``,
    ``distance_bias``, ``mix_heads``; ``value_norm_eps`` (0: values stored as projected).
    Tensors: ``q``, ``k``, ``v``, ``o`` (+ ``.b`` with ``bias``), ``r1``, ``r2`` [heads], ``talk`` [heads, heads]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.d, self.dv = int(p["head_dim"]), int(p.get("value_dim") or p["head_dim"])
        self.scale, self.chunk = float(p["scale"]), int(p.get("chunk") or 0)
        self.has_bias, self.distance_bias, self.mix_heads = bool(p.get("bias")), bool(p.get("distance_bias")), bool(p.get("mix_heads"))
        self.value_norm_eps = float(p.get("value_norm_eps") or 0.0)
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are no multiple of {self.kv_heads} kv heads")
        self.inner_width = self.heads * self.dv
        self.output_bias_spec = self.has_bias
        self.b_qkv = self.r1 = self.r2 = self.talk = self.output_bias = self.w_o = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H, G, d, dv = self.heads, self.kv_heads, self.d, self.dv
        out = {"q": TensorSpec((H * d, self.hidden)), "k": TensorSpec((G * d, self.hidden)),
               "v": TensorSpec((G * dv, self.hidden)), "o": TensorSpec((self.hidden, H * dv))}
        if self.has_bias:
            out.update({"q.b": TensorSpec((H * d,), "zeros_jitter"), "k.b": TensorSpec((G * d,), "zeros_jitter"),
                        "v.b": TensorSpec((G * dv,), "zeros_jitter"), "o.b": TensorSpec((self.hidden,), "zeros_jitter")})
        if self.distance_bias:
            out.update({"r1": TensorSpec((H,), "uniform", lo=0.0, hi=1.0), "r2": TensorSpec((H,), "uniform", lo=0.05, hi=1.0)})
        if self.mix_heads:
            out["talk"] = TensorSpec((H, H), "uniform", lo=-0.3, hi=0.7)
        return out

    def load(self, t) -> None:
        self.w_qkv = self._to_compute(torch.cat([t["q"], t["k"], t["v"]], dim=0))
        self.w_o = self._to_compute(t["o"])
        if self.has_bias:
            self.b_qkv = self._to_f32(torch.cat([t["q.b"], t["k.b"], t["v.b"]], dim=0))
            self.output_bias = self._to_f32(t["o.b"])
        if self.distance_bias:
            self.r1, self.r2 = self._to_f32(t["r1"]), self._to_f32(t["r2"])
        if self.mix_heads:
            self.talk = self._to_f32(t["talk"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="chunk" if self.chunk else "full", kv_heads=self.kv_heads, head_dim=self.d, window=self.chunk,
                         value_dim=self.dv if self.dv != self.d else 0)

    def write_inner(self, x, ctx, cache, out, column: int, scale: float) -> None:
        """The heads' outputs, times ``scale``, into columns ``column``.. of ``out`` [T, >= column + heads*value_dim]."""
        ops = self.rt.ops
        g = cache.group
        qkv = ops.linear(x, self.w_qkv)
        if cache.write:
            ops.kv_write_normed(qkv, self.b_qkv, g.slots, cache.kv, self.heads, self.kv_heads, self.d, self.dv, g.page_size,
                                self.value_norm_eps)
        ops.chunk_attention(qkv, self.b_qkv, cache.kv, g.block_table, ctx.tok_req, ctx.positions, self.heads, self.kv_heads,
                            self.d, self.dv, g.page_size, self.scale, self.chunk, self.r1, self.r2, self.talk, out, column, scale)

    def forward(self, x, ctx, cache):
        out = self.rt.ops.empty((x.shape[0], self.inner_width), self.rt.dtype)
        self.write_inner(x, ctx, cache, out, 0, 1.0)
        return self.rt.ops.linear(out, self.w_o)
