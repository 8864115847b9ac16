"""Mixture-of-experts feed-forward (``MoESpec``): every token uses the ``top`` experts its router scores
highest, out = sum over the chosen e of weight_e * down_e(relu(up_e x)^2).  The spec may ask for sigmoid scores,
weights that are not renormalised, weights that multiply an expert's input (out = sum expert_e(weight_e x)), gated
experts down_e(silu(gate_e x) * (up_e x)), whose gate and up matrices are then stacked expert by expert as
[gate_e; up_e] (or, ``act`` "glu_clamp", the clamped gate g sigmoid(slope g) (u + 1)), a bias on the router's logits,
and a shared expert that every token uses (a feed-forward part of its own, whatever kind its spec names, added to the
sum as it is or times sigmoid(w . x), one number a token; w then rides as one more row of the router's matrix).
An expert has no biases, so a weight on its input is a factor on the outputs of its first products: it is applied
to them in float32, inside the activation between the two products.

The router's logits are a float32 product and its softmax, choice and weights are float32
(``ops.moe_route``).  The experts' matrices are kept stacked: all up matrices one above the other and all
down matrices side by side.  A step of many rows runs two products over the stack, with the row's weight
for each expert (zero where it was not chosen) folded into the activation between them, so the experts a
token did not choose contribute exact zeros and nothing depends on where the rows of an expert lie; such
a step stays free of host reads, so single-token steps of many sequences replay from a graph.  A step of
few rows reads only the chosen experts' matrices (``ops.moe_rows``; with more (row, choice) pairs than
experts the pairs are sorted by expert on the device first, so that an expert's matrices are read once:
``ops.moe_rows_grouped``).  A prompt-sized step, which is never
replayed from a graph, sorts its (row, choice) pairs by expert, reads the experts' group sizes on the host
and runs one pair of products an expert on that expert's rows alone, so it does top / experts of the stacked
path's arithmetic.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .. import registry
from .base import FeedForward, Runtime, TensorDecl
from .swiglu import SwiGLU  # noqa: F401  (the shared expert's usual kind)


class MoE(FeedForward):
    capturable = True
    ROWS_SPARSE = 16      # up to this many rows a step reads only the chosen experts' matrices
    ROWS_GROUPED = 192    # from this many rows on a step runs every expert on its own rows (it reads their counts on the host)

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        decls = [TensorDecl(prefix + "router", (spec.experts, spec.hidden))]
        if getattr(spec, "router_bias", False):
            decls.append(TensorDecl(prefix + "router" + spec.router_bias_suffix, (spec.experts,), role="vector"))
        for e in range(spec.experts):
            if getattr(spec, "act", "relu2") != "relu2":
                decls.append(TensorDecl(prefix + f"e{e}.gate", (spec.intermediate, spec.hidden)))
            decls += [TensorDecl(prefix + f"e{e}.up", (spec.intermediate, spec.hidden)),
                      TensorDecl(prefix + f"e{e}.down", (spec.hidden, spec.intermediate))]
        shared = getattr(spec, "shared", None)
        if shared is not None:
            decls += registry.part_class("feed_forward", shared.kind).declare(shared, prefix + spec.shared_prefix)
            if getattr(spec, "shared_gate", False):
                decls.append(TensorDecl(prefix + spec.shared_prefix + spec.shared_gate_name, (1, spec.hidden)))
        return decls

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.act = getattr(spec, "act", "relu2")
        self.score = getattr(spec, "score", "softmax")
        self.renorm = bool(getattr(spec, "renorm", True))
        self.weight_input = getattr(spec, "weight_on", "output") == "input"
        self.limit, self.slope = float(getattr(spec, "act_limit", 0.0)), float(getattr(spec, "act_slope", 1.0))
        if self.act not in ("relu2", "swiglu", "glu_clamp") or self.score not in ("softmax", "sigmoid") or getattr(spec, "weight_on", "output") not in ("output", "input"):
            raise ValueError(f"{prefix}: unknown activation, score or weight placement in {spec}")
        ups = [tensors[prefix + f"e{e}.up"] for e in range(spec.experts)]
        if self.act != "relu2":      # a gated expert's rows: its gate matrix, then its up matrix
            ups = [t for e in range(spec.experts) for t in (tensors[prefix + f"e{e}.gate"], ups[e])]
        downs = [tensors[prefix + f"e{e}.down"] for e in range(spec.experts)]
        if len({t.dtype for t in ups + downs}) != 1:
            raise ValueError(f"{prefix}: the experts are stored in different dtypes; they must agree")
        self.up = torch.cat(ups, dim=0).contiguous()         # [experts * ff, hidden]
        self.down = torch.cat(downs, dim=1).contiguous()     # [hidden, experts * ff]
        self.router = tensors[prefix + "router"].contiguous()
        self.router_bias = None
        if getattr(spec, "router_bias", False):
            self.router_bias = tensors[prefix + "router" + spec.router_bias_suffix].to(torch.float32).contiguous()
        shared = getattr(spec, "shared", None)
        self.shared = None if shared is None else registry.part_class("feed_forward", shared.kind)(shared, prefix + spec.shared_prefix, tensors, runtime)
        self.shared_gated = shared is not None and bool(getattr(spec, "shared_gate", False))
        if self.shared_gated:
            # the gate's vector is one more row of the router's matrix: one product gives the logits and the gate's pre-activation
            gate = tensors[prefix + spec.shared_prefix + spec.shared_gate_name].reshape(1, spec.hidden).to(self.router.dtype)
            self.router = torch.cat([self.router, gate], dim=0).contiguous()
            if self.router_bias is not None:
                self.router_bias = torch.cat([self.router_bias, torch.zeros(1, dtype=torch.float32, device=self.router_bias.device)]).contiguous()

    def weight_bytes(self) -> int:
        """Bytes of the matrices a token's step reads: the router and the chosen experts."""
        per = (self.up.numel() + self.down.numel()) * self.up.element_size() // self.spec.experts
        shared = 0 if self.shared is None else self.shared.weight_bytes()
        return self.router.numel() * self.router.element_size() + per * self.spec.top + shared

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor) -> None:
        logits = self._experts(batch, x, out)
        if self.shared_gated:
            both = torch.empty_like(out)
            self.shared.forward(batch, x, both)
            self.rt.ops.add_rows_gated(out, both, logits[:, self.spec.experts])
            return
        if self.shared is not None:
            if out.dtype == torch.float32 and self.shared.adds_in_place(x.shape[0]):
                self.shared.forward_into(batch, x, out)     # its last product adds into the experts' sum
                return
            both = torch.empty_like(out)
            self.shared.forward(batch, x, both)
            self.rt.ops.add_rows(out, both)

    def _experts(self, batch, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """The chosen experts' weighted sum into ``out``; returns what the router's product left (the experts' logits and,
        behind them, the shared expert's gate pre-activation if there is one)."""
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        every = torch.empty((rows, self.router.shape[0]), dtype=torch.float32, device=x.device)
        ops.gemm(x, self.router, every, bias=self.router_bias)
        logits = every[:, :s.experts]
        kw = dict(kind=self.act, limit=self.limit, slope=self.slope)
        dense = torch.empty((rows, s.experts), dtype=torch.float32, device=x.device)
        index = torch.empty((rows, s.top), dtype=torch.int32, device=x.device)
        weight = torch.empty((rows, s.top), dtype=torch.float32, device=x.device)
        ops.moe_route(logits, s.top, float(s.renorm_eps), dense, index, weight, score=self.score, renorm=self.renorm)
        if rows <= self.ROWS_SPARSE and s.top < s.experts:
            if rows * s.top <= s.experts:      # hardly two pairs with one expert: a pair reads its expert's matrices
                ops.moe_rows(x, self.up, self.down, index, weight, out, s.experts, s.intermediate, weight_input=self.weight_input, **kw)
                return every
            # more pairs than experts: sorted by expert on the device, every expert's matrices are read once
            pairs = rows * s.top
            offsets = torch.empty(s.experts + 1, dtype=torch.int32, device=x.device)
            place = torch.empty(pairs, dtype=torch.int32, device=x.device)
            src_row = torch.empty(pairs, dtype=torch.int32, device=x.device)
            sorted_w = torch.empty(pairs, dtype=torch.float32, device=x.device) if self.weight_input else None
            ops.moe_group(index, s.experts, offsets, place, src_row, weight if self.weight_input else None, sorted_w)
            ys = torch.empty((pairs, s.hidden), dtype=torch.float32, device=x.device)
            ops.moe_rows_grouped(x, self.up, self.down, offsets, src_row, ys, s.experts, s.top, s.intermediate, sorted_weight=sorted_w, **kw)
            ops.moe_combine(ys, place, None if self.weight_input else weight, out, top=s.top)
            return every
        if rows >= self.ROWS_GROUPED and s.top < s.experts and (self._one_launch(x.dtype) or not torch.cuda.is_current_stream_capturing()):
            self._grouped(x, index, weight, out)
            return every
        up = torch.empty((rows, self.up.shape[0]), dtype=x.dtype, device=x.device)
        ops.gemm(x, self.up, up)
        act = up if self.act == "relu2" else torch.empty((rows, s.experts * s.intermediate), dtype=x.dtype, device=x.device)
        ops.moe_act(up, dense, act, s.experts, s.intermediate, weight_input=self.weight_input, **kw)
        ops.gemm(act, self.down, out)
        return every

    def _grouped(self, x: torch.Tensor, index: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
        """Every expert on its own rows: sort the pairs by expert, gather, two products over the groups, add up."""
        ops, s = self.rt.ops, self.spec
        rows, pairs, ff = x.shape[0], x.shape[0] * s.top, s.intermediate
        offsets = torch.empty(s.experts + 1, dtype=torch.int32, device=x.device)
        place = torch.empty(pairs, dtype=torch.int32, device=x.device)
        src_row = torch.empty(pairs, dtype=torch.int32, device=x.device)
        sorted_w = torch.empty(pairs, dtype=torch.float32, device=x.device) if self.weight_input else None
        ops.moe_group(index, s.experts, offsets, place, src_row, weight if self.weight_input else None, sorted_w)
        xs = torch.empty((pairs, s.hidden), dtype=x.dtype, device=x.device)
        ops.moe_gather(x, src_row, xs)
        per = self.up.shape[0] // s.experts     # rows of the stack an expert holds: ff, or gate and up
        one_launch = self._one_launch(x.dtype)
        bounds = None
        if one_launch and self.act != "relu2":
            # gate and up products, the pairs' weights and the activation in one kernel
            act = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
            ops.gemm_grouped(xs, self.up, act, offsets, s.experts, gated=True, row_weight=sorted_w, gate=self.act, limit=self.limit, slope=self.slope)
        else:
            act = torch.empty((pairs, per), dtype=x.dtype, device=x.device)
            if one_launch:
                ops.gemm_grouped(xs, self.up, act, offsets, s.experts)
            else:
                bounds = offsets.tolist()       # the one host read of such a step
                for e in range(s.experts):
                    lo, hi = bounds[e], bounds[e + 1]
                    if hi > lo:
                        ops.gemm_w_cols(xs[lo:hi], self.up[e * per:(e + 1) * per], act[lo:hi])
            if self.act == "relu2" and not self.weight_input:
                ops.relu2(act)
            else:
                # every sorted pair is a row of one "expert" here: its own weight (or 1), its own activation
                made = act if self.act == "relu2" else torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
                ops.moe_act(act, None if sorted_w is None else sorted_w.view(pairs, 1), made, 1, ff, kind=self.act, weight_input=self.weight_input,
                            limit=self.limit, slope=self.slope)
                act = made
        if one_launch:
            if s.top == 1 and self.weight_input:
                # every row has one pair and its weight is spent: the product's rows go straight to their places
                ops.gemm_grouped(act, self.down, out, offsets, s.experts, by_cols=True, row_map=src_row)
                return
            ys = torch.empty((pairs, s.hidden), dtype=torch.float32, device=x.device)
            ops.gemm_grouped(act, self.down, ys, offsets, s.experts, by_cols=True)
        else:
            ys = torch.empty((pairs, s.hidden), dtype=torch.float32, device=x.device)
            if bounds is None:
                bounds = offsets.tolist()
            for e in range(s.experts):
                lo, hi = bounds[e], bounds[e + 1]
                if hi > lo:
                    ops.gemm_w_cols(act[lo:hi], self.down[:, e * ff:(e + 1) * ff], ys[lo:hi])
        ops.moe_combine(ys, place, None if self.weight_input else weight, out, top=s.top)

    def _one_launch(self, act_dtype) -> bool:
        """Whether the tensor-core kernel that walks all groups in one launch takes this mixture's matrices."""
        ops, s = self.rt.ops, self.spec
        return (ops.gemm_grouped_fits(act_dtype, self.up, s.hidden, False) and ops.gemm_grouped_fits(act_dtype, self.down, s.intermediate, True))
