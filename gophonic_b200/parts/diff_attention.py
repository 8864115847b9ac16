"""Differential attention over the paged cache (``DiffAttentionSpec``): every query head has two softmax maps over the
same values; the head's output is the first map less lambda times the second, divided by its root mean square.

How it runs.  The two maps of every head are ordinary attention heads of ``head_dim`` whose keys are the two maps of
the head's key group, so the framework's attention kernels run them as 2 * heads query heads over 2 * kv_heads key
heads, with one option: two consecutive key heads read ONE value head (``v_share`` 2), which is how the cache keeps
the values once.  For the grouped-query arithmetic of those kernels (query head j reads key head j // group) the
rows of the query projection are reordered once, when the weights are loaded, so that a key group's query heads
stand as [map 1 of each head, map 2 of each head].  q | k | v is one product; the per-head-and-map RMS norm, the
rotation and the cache write are the row-wise kernel the other attention parts use; ``ops.diff_combine`` takes the
maps apart again and leaves the heads in the model's order for the output projection.  lambda is one number a layer,
computed once in float32 from the four learned vectors.
"""
from __future__ import annotations

import math
from typing import List, Mapping

import torch

from .. import registry
from .attention import choose_splits
from .base import KVRequest, Mixer, Runtime, TensorDecl


class DiffAttention(Mixer):
    capturable = True
    MAPS = 2

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        n = dict(spec.names)
        H, G, d, dv = spec.heads, spec.kv_heads, spec.head_dim, spec.value_dim
        decls = [TensorDecl(prefix + n["q"], (H * 2 * d, spec.hidden)), TensorDecl(prefix + n["k"], (G * 2 * d, spec.hidden)),
                 TensorDecl(prefix + n["v"], (G * dv, spec.hidden))]
        if spec.qk_norm is not None:
            decls += [TensorDecl(prefix + n["q_norm"], (d,), role="norm"), TensorDecl(prefix + n["k_norm"], (d,), role="norm")]
        decls += [TensorDecl(prefix + n[v], (d,), role="vector") for v in ("lq1", "lk1", "lq2", "lk2")]
        decls.append(TensorDecl(prefix + n["o"], (spec.hidden, H * dv)))
        return decls

    @classmethod
    def cache_request(cls, spec):
        # every key is kept (the mask is applied when they are read); a key group's two maps share its values
        return KVRequest(kv_heads=cls.MAPS * spec.kv_heads, head_dim=spec.head_dim, window=0, value_dim=spec.value_dim,
                         value_heads=spec.kv_heads)

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"{prefix}: {spec.heads} heads are not a multiple of {spec.kv_heads} kv heads")
        self.spec, self.rt = spec, runtime
        n = dict(spec.names)
        H, G, d, dv = spec.heads, spec.kv_heads, spec.head_dim, spec.value_dim
        self.per_group = H // G
        q, k, v = tensors[prefix + n["q"]], tensors[prefix + n["k"]], tensors[prefix + n["v"]]
        if not (q.dtype == k.dtype == v.dtype):
            raise ValueError(f"{prefix}: the projections are stored in different dtypes; they must agree")
        # [group][head of the group][map] -> [group][map][head of the group]
        q = q.view(G, self.per_group, self.MAPS, d, spec.hidden).permute(0, 2, 1, 3, 4).reshape(H * self.MAPS * d, spec.hidden)
        self.qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.o = tensors[prefix + n["o"]].contiguous()
        self.q_norm = self.k_norm = None
        self.norm_eps = 0.0
        if spec.qk_norm is not None:
            self.q_norm = tensors[prefix + n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm = tensors[prefix + n["k_norm"]].to(torch.float32).contiguous()
            self.norm_eps = float(spec.qk_norm.eps)
        f32 = lambda name: tensors[prefix + n[name]].to(torch.float32)
        lam = torch.exp((f32("lq1") * f32("lk1")).sum()) - torch.exp((f32("lq2") * f32("lk2")).sum()) + torch.tensor(
            float(spec.lambda_init), dtype=torch.float32, device=self.o.device)
        self.lam = float(lam.item())
        if not math.isfinite(self.lam):
            raise ValueError(f"{prefix}: the factor of the second map is {self.lam}")
        self.position = registry.part_class("position", spec.position.kind)(spec.position, prefix, tensors, runtime)
        self.q_heads, self.k_heads = self.MAPS * H, self.MAPS * G
        self.q_dim = self.q_heads * d

    def weight_bytes(self) -> int:
        return self.qkv.numel() * self.qkv.element_size() + self.o.numel() * self.o.element_size()

    def prepare(self, capacity: int) -> None:
        self.position.prepare(capacity)

    def _seen(self, max_kv_len: int) -> int:
        s = self.spec
        seen = max_kv_len
        for size in (s.chunk, s.window):
            if size > 0:
                seen = min(seen, size)
        return seen

    def plan(self, nseq: int, max_q_len: int, max_kv_len: int, sm_count: int):
        """Single-token steps cut the keys a row can see (at most its block or window) into pieces."""
        if max_q_len != 1:
            return 1
        elem = 4 if self.rt.is_fp32 else 2
        page_bytes = 64 * (self.spec.head_dim + self.spec.value_dim) * elem
        return choose_splits(nseq * self.k_heads, self._seen(max_kv_len), sm_count, page_bytes)

    def key_splits(self, batch):
        s = self.spec
        splits = int(batch.plan_for(self) or 1)
        if splits <= 1:
            return 1, None
        return splits, batch.workspace(("attention key splits", self.q_heads, s.value_dim, splits),
                                       self.rt.ops.attention_scratch_floats(batch.nseq, self.q_heads, s.value_dim, splits))

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor, cache) -> None:
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        if cache is None:
            raise ValueError("attention needs a key/value cache plane")
        if cache.k.dtype != x.dtype:
            raise ValueError(f"attention: cache holds {cache.k.dtype}, activations are {x.dtype}")
        qkv = torch.empty((rows, self.qkv.shape[0]), dtype=x.dtype, device=x.device)
        ops.gemm(x, self.qkv, qkv)
        cos, sin, rot = self.position.kernel_args()
        ops.qk_norm_rope_kv_write(qkv, self.q_heads, self.k_heads, s.head_dim, self.q_norm, self.k_norm, self.norm_eps, cos, sin, rot,
                                  batch.row_pos, batch.row_seq, batch.seq_slot, cache.block_table, cache.k, cache.v, cache.writable,
                                  pairs=bool(getattr(self.position, "pairs", False)), value_dim=s.value_dim, v_share=self.MAPS)
        maps = torch.empty((rows, self.q_heads * s.value_dim), dtype=x.dtype, device=x.device)
        splits, scratch = self.key_splits(batch)
        ops.attention(qkv, maps, cache.k, cache.v, cache.block_table, batch.seq_slot, batch.seq_q_start, batch.seq_q_len, batch.seq_kv_len,
                      batch.nseq, batch.max_q_len, self.q_heads, self.k_heads, s.head_dim, float(s.scale), int(s.window), splits, scratch,
                      value_dim=s.value_dim, chunk=int(s.chunk), v_share=self.MAPS)
        ctx = torch.empty((rows, s.heads * s.value_dim), dtype=x.dtype, device=x.device)
        ops.diff_combine(maps, ctx, s.heads, self.per_group, s.value_dim, self.lam, float(s.eps), 1.0 - float(s.lambda_init))
        ops.gemm(ctx, self.o, out)
