"""Dense feed-forwards beside the gated SiLU one.

``ReluSquared`` (``ReluSquaredSpec``): out = down(relu(up(x))^2).
``ClampedGLU`` (``ClampedGLUSpec``): out = down(g sigmoid(slope g) (u + 1)) with g = min(gate(x), limit) and
u = clamp(up(x), -limit, limit); gate and up are one product, the activation is computed in float32.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .base import FeedForward, Runtime, TensorDecl


class ReluSquared(FeedForward):
    capturable = True

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        up, down = spec.names
        return [TensorDecl(prefix + up, (spec.intermediate, spec.hidden)), TensorDecl(prefix + down, (spec.hidden, spec.intermediate))]

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec, self.rt = spec, runtime
        self.up = tensors[prefix + spec.names[0]].contiguous()
        self.down = tensors[prefix + spec.names[1]].contiguous()

    def weight_bytes(self) -> int:
        return self.up.numel() * self.up.element_size() + self.down.numel() * self.down.element_size()

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor) -> None:
        ops = self.rt.ops
        act = torch.empty((x.shape[0], self.spec.intermediate), dtype=x.dtype, device=x.device)
        ops.gemm(x, self.up, act)
        ops.relu2(act)
        ops.gemm(act, self.down, out)


class ClampedGLU(FeedForward):
    capturable = True

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        gate, up, down = spec.names
        return [TensorDecl(prefix + gate, (spec.intermediate, spec.hidden)), TensorDecl(prefix + up, (spec.intermediate, spec.hidden)),
                TensorDecl(prefix + down, (spec.hidden, spec.intermediate))]

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec, self.rt = spec, runtime
        gate, up = tensors[prefix + spec.names[0]], tensors[prefix + spec.names[1]]
        if gate.dtype != up.dtype:
            raise ValueError(f"{prefix}: gate is {gate.dtype} and up is {up.dtype}; they must agree")
        self.gate_up = torch.cat([gate, up], dim=0).contiguous()      # one product reads x once: gate rows, then up rows
        self.down = tensors[prefix + spec.names[2]].contiguous()

    def weight_bytes(self) -> int:
        return self.gate_up.numel() * self.gate_up.element_size() + self.down.numel() * self.down.element_size()

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor) -> None:
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        gu = torch.empty((rows, 2 * s.intermediate), dtype=x.dtype, device=x.device)
        ops.gemm(x, self.gate_up, gu)
        act = torch.empty((rows, s.intermediate), dtype=x.dtype, device=x.device)
        ops.moe_act(gu, None, act, 1, s.intermediate, kind="glu_clamp", limit=float(s.limit), slope=float(s.slope))
        ops.gemm(act, self.down, out)
