"""RMSNorm part: y = x * (1 / sqrt(mean(x^2) + eps)) * weight, plain weight
(internal/qwen3lm/ops.go:251-254; kernels_scalar.go:15-35), or, where the spec gives an ``offset``, a
tensor that holds the weight less that offset: y = ... * (offset + w).  Statistics are fp32; the weight is held in fp32
(an exact widening of a bfloat16 checkpoint vector, the offset added in fp32)."""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .base import Norm, Runtime, TensorDecl


class RMSNorm(Norm):
    capturable = True

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        # a tensor that holds a difference from the offset is initialised near zero
        role = "vector" if float(getattr(spec, "offset", 0.0)) != 0.0 else "norm"
        return [TensorDecl(prefix + getattr(spec, "tensor", "weight"), (spec.size,), role=role)]

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.weight = tensors[prefix + getattr(spec, "tensor", "weight")].to(torch.float32).contiguous()
        offset = float(getattr(spec, "offset", 0.0))
        if offset != 0.0:
            self.weight = (self.weight + offset).contiguous()
        gain = float(getattr(spec, "gain", 1.0))
        if gain != 1.0:
            self.weight = (self.weight * gain).contiguous()
        self.eps = float(spec.eps)

    def rms_fold(self):
        return self.weight, self.eps

    def forward(self, h: torch.Tensor, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> None:
        self.rt.ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)
