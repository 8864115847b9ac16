"""Junction ``reinject`` (``ReinjectSpec``): where a pass through repeated layers begins, the residual is mixed
with the embedding output and the pass's own vector is added,

    x <- W [x; x0] + steps[index].

One row-wise kernel lays the residual (with whatever addend is still owed to it) and x0 side by side in the
activation dtype, one product makes the new float32 residual and adds the vector (in its epilogue for prompt-sized
steps, by a row-wise kernel otherwise).  The old
residual is not needed afterwards.  A junction is built once per schedule position that names it; positions that
name the same tensors share them.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .base import Part, Runtime, TensorDecl


class Reinject(Part):
    category = "junction"
    capturable = True

    @classmethod
    def declare(cls, spec, prefix: str = "") -> List[TensorDecl]:
        return [TensorDecl(prefix + spec.weight, (spec.hidden, 2 * spec.hidden)),
                TensorDecl(prefix + spec.steps, (spec.passes, spec.hidden), role="vector")]

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        if not 0 <= spec.index < spec.passes:
            raise ValueError(f"reinject: pass {spec.index} of {spec.passes}")
        self.spec = spec
        self.rt = runtime
        self.weight = tensors[prefix + spec.weight].contiguous()
        self.step = tensors[prefix + spec.steps][spec.index].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, batch, h: torch.Tensor, pending, x0: torch.Tensor):
        """``h``: the float32 residual, ``pending``: a float32 addend still owed to it (anything else: nothing owed),
        ``x0``: the embedding output.  Returns the new residual, to which nothing is owed."""
        ops = self.rt.ops
        rows, hidden = h.shape
        joined = torch.empty((rows, 2 * hidden), dtype=self.rt.act_dtype, device=h.device)
        ops.concat_cast(h, pending if isinstance(pending, torch.Tensor) else None, x0, joined)
        out = torch.empty((rows, hidden), dtype=torch.float32, device=h.device)
        ops.gemm(joined, self.weight, out, bias=self.step)
        return out
