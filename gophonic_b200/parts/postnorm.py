"""A block whose sublayers read the residual itself and whose norms stand behind them (``PostNormLayerSpec``):

    x <- x + mult * scale_1 * norm_1(mixer(x));    x <- x + mult * scale_2 * norm_2(feed_forward(x))

The norm is the registered norm of the spec (an ``RMSNorm``, whose weight already holds its offset and gain); the
block folds ``mult`` and the sublayer's scale vector into that weight once, in float32, so a sublayer's output enters
the residual in one kernel: statistics of the output, the scaled norm, the float32 add, and the new rows once more
in the activation dtype for the sublayer that reads them next (``ops.norm_scale_add``).  The residual stays float32;
what a sublayer reads in bfloat16 mode is its rounding.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .. import registry
from .base import ActRows, Part, Runtime, TensorDecl


class PostNormBlock(Part):
    category = "block"

    @classmethod
    def _sublayers(cls, layer):
        out = [("mixer", layer.mixer, layer.mixer_prefix, layer.mixer_norm, layer.mixer_norm_prefix, 0)]
        if layer.feed_forward is not None:
            out.append(("feed_forward", layer.feed_forward, layer.feed_forward_prefix, layer.feed_forward_norm, layer.feed_forward_norm_prefix, 1))
        return out

    @classmethod
    def declare(cls, layer, prefix: str = "") -> List[TensorDecl]:
        p = layer.prefix
        decls: List[TensorDecl] = []
        for category, spec, sub_prefix, norm, norm_prefix, q in cls._sublayers(layer):
            decls += registry.part_class("norm", norm.kind).declare(norm, p + norm_prefix)
            decls += registry.part_class(category, spec.kind).declare(spec, p + sub_prefix)
            if layer.scale_names is not None:
                decls.append(TensorDecl(p + layer.scale_names[q], (norm.size,), role="norm"))
        return decls

    def __init__(self, layer, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        p = layer.prefix
        self.layer = layer
        self.rt = runtime
        self.parts, self.norms, self.weights = [], [], []
        for category, spec, sub_prefix, norm, norm_prefix, q in self._sublayers(layer):
            n = registry.part_class("norm", norm.kind)(norm, p + norm_prefix, tensors, runtime)
            fold = n.rms_fold()
            if fold is None:
                raise ValueError(f"{p}{norm_prefix}: a norm behind a sublayer must be an RMS norm with a float32 weight")
            w = fold[0].to(torch.float32) * float(layer.residual_mult)
            if layer.scale_names is not None:
                w = w * tensors[p + layer.scale_names[q]].to(torch.float32)
            self.norms.append(n)
            self.weights.append((w.contiguous(), float(fold[1])))
            self.parts.append(registry.part_class(category, spec.kind)(spec, p + sub_prefix, tensors, runtime))
        self.mixer = self.parts[0]
        self.feed_forward = self.parts[1] if len(self.parts) > 1 else None

    @classmethod
    def cache_request(cls, layer):
        return registry.part_class("mixer", layer.mixer.kind).cache_request(layer.mixer)

    def prepare(self, capacity: int) -> None:
        self.mixer.prepare(capacity)

    def mixers(self) -> List[Part]:
        return [self.mixer]

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts if hasattr(p, "weight_bytes"))

    @property
    def capturable(self) -> bool:
        return all(p.capturable for p in self.parts + self.norms)

    def forward(self, batch, h: torch.Tensor, pending, cache):
        """Runs the layer on residual ``h`` (float32, updated in place).  ``pending``: a float32 addend still owed to the
        residual, ``ActRows`` (the residual's rows in the activation dtype), or anything else (nothing known)."""
        ops = self.rt.ops
        rows, hidden = h.shape
        act = self.rt.act_dtype
        if isinstance(pending, torch.Tensor):
            ops.add_rows(h, pending)
        x = h
        if act != torch.float32:
            if isinstance(pending, ActRows):
                x = pending.x
            else:
                x = torch.empty((rows, hidden), dtype=act, device=h.device)
                ops.f32_to_bf16(h, x)
        y = torch.empty((rows, hidden), dtype=torch.float32, device=h.device)
        for q, part in enumerate(self.parts):
            if q == 0:
                part.forward(batch, x, y, cache)
            else:
                part.forward(batch, x, y)
            w, eps = self.weights[q]
            if act != torch.float32:
                x_next = torch.empty((rows, hidden), dtype=act, device=h.device)
                ops.norm_scale_add(h, y, w, eps, x_next)
                x = x_next
            else:
                ops.norm_scale_add(h, y, w, eps)     # the next sublayer reads h itself
        return ActRows(x) if act != torch.float32 else None
