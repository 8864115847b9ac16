"""Grouped-query attention with a kept-first-tokens window, a softmax sink (a unit, or a learned score
per head), biased projections, a norm of q and k (per head, or over the whole projection), an output gate
and, optionally, another layer's keys and values (``GatedAttentionSpec``); each of them can be left off.

Per row: q | k | v | g = x [Wq; Wk; Wv; Wg]^T in one product (a layer that reads another layer's
cache has only q and g); biases, the norm of q and k, their position encoding and the cache write in
one row-wise kernel; scores (q . k) * scale in float32 over the keys j <= i with i - j < window or
j < keep_first, softmax with one more term in the denominator; the heads, each ``value_dim`` wide,
times sigmoid(g); out = ctx Wo^T (+ bo).  Keys are cached after rotation, so a layer that shares them
rotates only its queries.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .. import registry
from .attention import Attention
from .base import KVRequest, Runtime, TensorDecl


class GatedAttention(Attention):
    capturable = True

    @staticmethod
    def _names(spec):
        return dict(spec.names)

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        n = cls._names(spec)
        qd, kd, vd = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim, spec.kv_heads * spec.value_dim
        od = spec.heads * spec.value_dim
        decls = [TensorDecl(prefix + n["q"], (qd, spec.hidden))]
        if spec.bias:
            decls.append(TensorDecl(prefix + n["q"] + spec.bias_suffix, (qd,), role="vector"))
        if spec.own_kv:
            decls += [TensorDecl(prefix + n["k"], (kd, spec.hidden)), TensorDecl(prefix + n["v"], (vd, spec.hidden))]
            if spec.bias:
                decls += [TensorDecl(prefix + n["k"] + spec.bias_suffix, (kd,), role="vector"),
                          TensorDecl(prefix + n["v"] + spec.bias_suffix, (vd,), role="vector")]
        if spec.gate:
            decls.append(TensorDecl(prefix + n["g"], (od, spec.hidden)))
        if getattr(spec, "qk_norm", None) is not None:
            span = bool(getattr(spec, "qk_norm_span", False))
            decls.append(TensorDecl(prefix + n["q_norm"], (qd if span else spec.head_dim,), role="norm"))
            if spec.own_kv:
                decls.append(TensorDecl(prefix + n["k_norm"], (kd if span else spec.head_dim,), role="norm"))
        if getattr(spec, "sink_learned", False):
            decls.append(TensorDecl(prefix + n["sink"], (spec.heads,), role="vector"))
        decls.append(TensorDecl(prefix + n["o"], (spec.hidden, od)))
        if getattr(spec, "out_bias", False):
            decls.append(TensorDecl(prefix + n["o"] + spec.bias_suffix, (spec.hidden,), role="vector"))
        return decls

    @classmethod
    def cache_request(cls, spec):
        # every key is kept (the window is a mask), so layers with different windows share a group
        return KVRequest(kv_heads=spec.kv_heads, head_dim=spec.head_dim, window=0, value_dim=spec.value_dim)

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"{prefix}: {spec.heads} heads are not a multiple of {spec.kv_heads} kv heads")
        self.spec = spec
        self.rt = runtime
        n = self._names(spec)
        parts = [tensors[prefix + n["q"]]]
        if spec.own_kv:
            parts += [tensors[prefix + n["k"]], tensors[prefix + n["v"]]]
        if spec.gate:
            parts.append(tensors[prefix + n["g"]])
        if len({t.dtype for t in parts}) != 1:
            raise ValueError(f"{prefix}: the projections are stored in different dtypes; they must agree")
        self.qkv = torch.cat(parts, dim=0).contiguous()     # q | k | v | g: one product reads x once
        self.o = tensors[prefix + n["o"]].contiguous()
        f32 = lambda name: tensors[prefix + name + spec.bias_suffix].to(torch.float32).contiguous()
        self.biases = None
        if spec.bias:
            self.biases = (f32(n["q"]), f32(n["k"]) if spec.own_kv else None, f32(n["v"]) if spec.own_kv else None)
        # the norm of q and k (float32 weights; with ``qk_norm_span`` one weight over all heads), the learned sink
        # scores and the output projection's bias
        self.q_norm = self.k_norm = self.sinks = self.o_bias = None
        self.eps = 0.0
        self.norm_span = bool(getattr(spec, "qk_norm_span", False))
        if getattr(spec, "qk_norm", None) is not None:
            self.q_norm = tensors[prefix + n["q_norm"]].to(torch.float32).contiguous()
            if spec.own_kv:
                self.k_norm = tensors[prefix + n["k_norm"]].to(torch.float32).contiguous()
            self.eps = float(spec.qk_norm.eps)
        if getattr(spec, "sink_learned", False):
            self.sinks = tensors[prefix + n["sink"]].to(torch.float32).contiguous()
        if getattr(spec, "out_bias", False):
            self.o_bias = tensors[prefix + n["o"] + spec.bias_suffix].to(torch.float32).contiguous()
        self.position = registry.part_class("position", spec.position.kind)(spec.position, prefix, tensors, runtime)
        self.q_dim = spec.heads * spec.head_dim
        self.kv_heads_own = spec.kv_heads if spec.own_kv else 0
        self.k_dim = self.kv_heads_own * spec.head_dim
        self.v_dim = self.kv_heads_own * spec.value_dim
        self.o_dim = spec.heads * spec.value_dim
        self.g_off = self.q_dim + self.k_dim + self.v_dim

    # prompt-sized steps: the output projection adds into the float32 residual in its own epilogue
    # (the folded decode path of the plain attention part is not offered)
    def adds_in_place(self, rows: int) -> bool:
        ops = self.rt.ops
        return (self.o.dtype == torch.bfloat16 and self.rt.act_dtype == torch.bfloat16 and self.o_dim % 8 == 0
                and self.spec.hidden % 4 == 0 and ops.gemm_algo(rows, self.spec.hidden, self.o_dim) == "tc5_pair")

    def forward_into(self, batch, x: torch.Tensor, h: torch.Tensor, cache) -> None:
        self.rt.ops.gemm_add(self._gated_heads(batch, x, cache), self.o, h, bias=self.o_bias)

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor, cache) -> None:
        self.rt.ops.gemm(self._gated_heads(batch, x, cache), self.o, out, bias=self.o_bias)

    def folds_norm(self, rows: int, norm) -> bool:
        return False

    def plan(self, nseq: int, max_q_len: int, max_kv_len: int, sm_count: int):
        """Single-token steps cut the keys a row can see (the window and the kept first tokens) into pieces."""
        if max_q_len != 1:
            return 1
        s = self.spec
        seen = min(max_kv_len, s.window + s.keep_first) if s.window > 0 else max_kv_len
        return super().plan(nseq, max_q_len, seen, sm_count)

    def key_splits(self, batch):
        s = self.spec
        splits = int(batch.plan_for(self) or 1)
        if splits <= 1:
            return 1, None
        return splits, batch.workspace(("attention key splits", s.heads, s.value_dim, splits),
                                       self.rt.ops.attention_scratch_floats(batch.nseq, s.heads, s.value_dim, splits))

    def _gated_heads(self, batch, x: torch.Tensor, cache) -> torch.Tensor:
        """Everything up to the output projection: [rows, heads * value_dim] in the activation dtype."""
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        if cache is None:
            raise ValueError("attention needs a key/value cache plane")
        if cache.k.dtype != x.dtype:
            raise ValueError(f"attention: cache holds {cache.k.dtype}, activations are {x.dtype}")
        if cache.writable != s.own_kv:
            raise ValueError("attention: a layer with keys of its own writes its cache plane, a layer without reads another's")
        qkvg = torch.empty((rows, self.qkv.shape[0]), dtype=x.dtype, device=x.device)
        ops.gemm(x, self.qkv, qkvg)
        cos, sin, rot = self.position.kernel_args()
        ops.qk_norm_rope_kv_write(qkvg, s.heads, self.kv_heads_own, s.head_dim, self.q_norm, self.k_norm, self.eps, cos, sin, rot,
                                  batch.row_pos, batch.row_seq, batch.seq_slot, cache.block_table, cache.k if s.own_kv else None,
                                  cache.v if s.own_kv else None, s.own_kv, biases=self.biases,
                                  pairs=bool(getattr(self.position, "pairs", False)), value_dim=s.value_dim, span=self.norm_span)
        ctx = torch.empty((rows, self.o_dim), dtype=x.dtype, device=x.device)
        splits, scratch = self.key_splits(batch)
        ops.attention(qkvg, ctx, cache.k, cache.v, cache.block_table, batch.seq_slot, batch.seq_q_start, batch.seq_q_len,
                      batch.seq_kv_len, batch.nseq, batch.max_q_len, s.heads, s.kv_heads, s.head_dim, float(s.scale), int(s.window),
                      splits, scratch, value_dim=s.value_dim, keep_first=int(s.keep_first), sink=bool(s.sink) or self.sinks is not None,
                      sinks=self.sinks)
        if s.gate:
            ops.head_norm_gate(ctx, qkvg[:, self.g_off:self.g_off + self.o_dim], ctx, s.heads, s.value_dim, ops.GATE_SIGMOID)
        return ctx
