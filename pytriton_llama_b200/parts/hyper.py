"""Several copies of the residual stream with learned reads and writes (hyper-connections).

The stream is S copies x_1 .. x_S, float32 [T, S, width], all equal to the embedding output at the
start.  A sub-layer reads u = sum_s read[s] x_s through an RMS norm and its output y is written back
to all copies at once, from the old ones:

    x_t <- sum_s mix[s, t] x_s + mult * out[t] * y

At the end of the model the copies are summed (a read of ones).  One copy with read = mix = out = 1
is the plain residual sum x <- x + mult * y, and that is how a model without copies runs here.

The write of a sub-layer and the read + norm of the next one are a single operator
(``ops.stream_mix_norm``): the block hands the pending write on as a ``StreamUpdate`` and the norm
that reads the stream next applies it, as the plain pre-norm block hands on its un-added output.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .base import Part, PartSpec, Runtime, TensorSpec, build_part, register_part


@dataclass
class StreamUpdate:
    """The output of a sub-layer that is still to be written to the copies of the stream."""
    y: torch.Tensor                 # [T, width], compute type or float32
    mix: torch.Tensor               # float32 [S, S], indexed [from, to]
    out: torch.Tensor               # float32 [S], the residual multiplier folded in


@register_part("norm", "stream_rmsnorm")
class StreamRMSNorm(Part):
    """params: ``width``, ``eps``, ``streams``, ``learned`` (a ``read`` tensor [streams]; else a read of ones).
    Tensors: ``weight`` [width], ``read`` [streams]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width, self.eps, self.streams = int(p["width"]), float(p["eps"]), int(p["streams"])
        self.learned = bool(p.get("learned", False))
        self.weight: Optional[torch.Tensor] = None
        self.read: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out = {"weight": TensorSpec((self.width,), init=self.spec.params.get("init", "ones"))}
        if self.learned:
            out["read"] = TensorSpec((self.streams,), "uniform", lo=0.2, hi=0.6)
        return out

    def load(self, tensors) -> None:
        self.weight = self._to_f32(tensors["weight"])
        self.read = self._to_f32(tensors["read"]) if self.learned else torch.ones(self.streams, dtype=torch.float32, device=self.rt.device)

    def forward(self, x, residual, rows=None):
        """``x``: the embedding output when ``residual`` is None (the copies start from it), else the
        ``StreamUpdate`` of the sub-layer before, or None.  ``residual``: the copies, float32 [T, S, width]."""
        ops = self.rt.ops
        if residual is None:
            return ops.stream_mix_norm(None, x, None, None, None, self.read, self.weight, self.eps, self.streams, rows, self.rt.dtype)
        if x is None:
            return ops.stream_mix_norm(residual, None, None, None, None, self.read, self.weight, self.eps, self.streams, rows, self.rt.dtype)
        return ops.stream_mix_norm(residual, None, x.y, x.mix, x.out, self.read, self.weight, self.eps, self.streams, rows, self.rt.dtype)


@register_part("block", "hyper_connections")
class HyperConnectionBlock(Part):
    """params: ``streams``, ``mult`` (the residual multiplier), ``learned``.  Nested parts: ``norm1``, ``mixer``;
    ``norm2`` and ``ffn`` (both or neither).  Tensors (``learned``): ``mix1``, ``mix2`` [streams, streams] indexed
    [from, to], ``out1``, ``out2`` [streams]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.streams, self.mult, self.learned = int(p["streams"]), float(p.get("mult", 1.0)), bool(p.get("learned", False))
        self.norm1 = build_part("norm", spec.parts["norm1"], runtime)
        self.mixer = build_part("mixer", spec.parts["mixer"], runtime)
        if ("norm2" in spec.parts) != ("ffn" in spec.parts):
            raise ValueError("a block has both norm2 and ffn, or neither")
        self.norm2 = build_part("norm", spec.parts["norm2"], runtime) if "norm2" in spec.parts else None
        self.ffn = build_part("ffn", spec.parts["ffn"], runtime) if "ffn" in spec.parts else None
        self.mix = [None, None]
        self.out = [None, None]

    def children(self):
        parts = {"norm1": self.norm1, "mixer": self.mixer, "norm2": self.norm2, "ffn": self.ffn}
        return {k: v for k, v in parts.items() if v is not None}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        if not self.learned:
            return {}
        S = self.streams
        out = {"mix1": TensorSpec((S, S), "uniform", lo=0.0, hi=0.6), "out1": TensorSpec((S,), "uniform", lo=0.3, hi=1.0)}
        if self.ffn is not None:
            out.update({"mix2": TensorSpec((S, S), "uniform", lo=0.0, hi=0.6), "out2": TensorSpec((S,), "uniform", lo=0.3, hi=1.0)})
        return out

    def load(self, tensors) -> None:
        for q in (0, 1):
            if q == 1 and self.ffn is None:
                continue
            self.mix[q] = self._to_f32(tensors[f"mix{q + 1}"])
            self.out[q] = (self._to_f32(tensors[f"out{q + 1}"]) * self.mult).contiguous()

    def after_load(self) -> None:
        if not self.learned:
            dev = self.rt.device
            for q in (0, 1):
                self.mix[q] = torch.eye(self.streams, dtype=torch.float32, device=dev)
                self.out[q] = torch.full((self.streams,), self.mult, dtype=torch.float32, device=dev)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, x, residual, ctx, cache):
        y, residual = self.norm1.forward(x, residual)
        pending = StreamUpdate(self.mixer.forward(y, ctx, cache), self.mix[0], self.out[0])
        if self.ffn is not None:
            y, residual = self.norm2.forward(pending, residual)
            pending = StreamUpdate(self.ffn.forward(y), self.mix[1], self.out[1])
        return pending, residual
