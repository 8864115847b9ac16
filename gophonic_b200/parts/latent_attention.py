"""Latent attention over the paged cache (``LatentAttentionSpec``): queries, keys and values are made from low-rank
latents and only the key/value latent c and one rotated key part k_r are cached, kv_rank + rot_dim numbers a token.

How it runs.  A head's plain key is W_uk c and its value W_uv c, so a score is q_plain . (W_uk c) + q_rot . k_r =
(W_uk^T q_plain) . c + q_rot . k_r and a head's output is W_uv (sum_j p_j c_j): the products with W_uk and W_uv move
from the keys to the queries and to the outputs, and attention itself runs over the cache as it is, as one key head of
kv_rank + rot_dim channels that all query heads read and whose first kv_rank channels are also the values (the
cache keeps no value plane: ``KVRequest.values_in_keys``).  Nothing is expanded per cached token, so prompts in
portions, single tokens and batches are one path.

Per step: one product for both down-projections; a row-wise kernel for the two RMS norms, the rotation of k_r and the
cache write (``ops.latent_prep``); the query up-projection; the per-head product with W_uk and the rotation of the
queries' rotated part into the absorbed queries; attention; the per-head product with W_uv; the output projection.
The per-head products are one launch for all heads: on the CUDA cores for few rows and for float32, on the tensor cores
(mma.sync) for prompts in bfloat16; operands that kernel cannot take run one product a head.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .. import registry
from .attention import choose_splits
from .base import KVRequest, Mixer, Runtime, TensorDecl


class LatentAttention(Mixer):
    capturable = True
    ROWS_ONE_LAUNCH = 32      # up to this many rows the per-head products run as one launch for all heads

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        n = dict(spec.names)
        H, d, dr, dv, Q, R = spec.heads, spec.head_dim, spec.rot_dim, spec.value_dim, spec.q_rank, spec.kv_rank
        return [TensorDecl(prefix + n["dq"], (Q, spec.hidden)), TensorDecl(prefix + n["dq_norm"], (Q,), role="norm"),
                TensorDecl(prefix + n["uq"], (H * (d + dr), Q)), TensorDecl(prefix + n["dkv"], (R + dr, spec.hidden)),
                TensorDecl(prefix + n["dkv_norm"], (R,), role="norm"), TensorDecl(prefix + n["uk"], (H * d, R)),
                TensorDecl(prefix + n["uv"], (H * dv, R)), TensorDecl(prefix + n["o"], (spec.hidden, H * dv))]

    @classmethod
    def cache_request(cls, spec):
        return KVRequest(kv_heads=1, head_dim=spec.kv_rank + spec.rot_dim, window=0, value_dim=spec.kv_rank, values_in_keys=True)

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec, self.rt = spec, runtime
        n = dict(spec.names)
        H, d, dv, R = spec.heads, spec.head_dim, spec.value_dim, spec.kv_rank
        dq, dkv = tensors[prefix + n["dq"]], tensors[prefix + n["dkv"]]
        if dq.dtype != dkv.dtype:
            raise ValueError(f"{prefix}: the down-projections are stored as {dq.dtype} and {dkv.dtype}; they must agree")
        self.down = torch.cat([dq, dkv], dim=0).contiguous()          # x is read once
        self.uq = tensors[prefix + n["uq"]].contiguous()
        uk, uv = tensors[prefix + n["uk"]], tensors[prefix + n["uv"]]
        # a head's W_uk is [head_dim, kv_rank]: as stored it maps plain query channels (K) to latent channels (N)
        self.uk_kn = uk.view(H, d, R).contiguous()
        self.uk_nk = self.uk_kn.transpose(1, 2).contiguous()          # [heads, kv_rank, head_dim] for a product a head
        self.uv_nk = uv.view(H, dv, R).contiguous()                   # as stored: latent channels (K) to value channels (N)
        self.uv_kn = self.uv_nk.transpose(1, 2).contiguous()
        self.o = tensors[prefix + n["o"]].contiguous()
        self.q_norm = tensors[prefix + n["dq_norm"]].to(torch.float32).contiguous()
        self.kv_norm = tensors[prefix + n["dkv_norm"]].to(torch.float32).contiguous()
        self.position = registry.part_class("position", spec.position.kind)(spec.position, prefix, tensors, runtime)
        if spec.rot_dim > 0 and not getattr(self.position, "pairs", False):
            raise ValueError(f"{prefix}: the rotated key part turns neighbouring channels together; position kind '{spec.position.kind}' does not")
        self.key_dim = R + spec.rot_dim

    def weight_bytes(self) -> int:
        ts = (self.down, self.uq, self.uk_kn, self.uv_nk, self.o)
        return sum(t.numel() * t.element_size() for t in ts)

    def prepare(self, capacity: int) -> None:
        self.position.prepare(capacity)

    def plan(self, nseq: int, max_q_len: int, max_kv_len: int, sm_count: int):
        if max_q_len != 1:
            return 1
        s = self.spec
        seen = max_kv_len
        for size in (s.chunk, s.window):
            if size > 0:
                seen = min(seen, size)
        elem = 4 if self.rt.is_fp32 else 2
        # a page of latents fills most of an SM's shared memory twice over: one CTA an SM, where the model of the split
        # choice counts two
        return choose_splits(nseq, seen, max(1, sm_count // 2), 64 * self.key_dim * elem)

    def key_splits(self, batch):
        s = self.spec
        splits = int(batch.plan_for(self) or 1)
        if splits <= 1:
            return 1, None
        return splits, batch.workspace(("attention key splits", s.heads, s.kv_rank, splits),
                                       self.rt.ops.attention_scratch_floats(batch.nseq, s.heads, s.kv_rank, splits))

    def _per_head(self, a: torch.Tensor, w_kn: torch.Tensor, w_nk: torch.Tensor, out: torch.Tensor) -> None:
        """out[:, h, :] = a[:, h, :] @ w_kn[h] for every head (``w_nk`` holds the same matrices transposed)."""
        ops = self.rt.ops
        rows, heads, K = a.shape
        if (self.rt.is_fp32 or rows <= self.ROWS_ONE_LAUNCH) and K <= ops.HEAD_GEMM_MAX_K:
            ops.head_gemm(a, w_kn, out)
            return
        if ops.head_gemm_mma_accepts(a, w_nk, out):
            ops.head_gemm_mma(a, w_nk, out)
            return
        for h in range(heads):
            ops.gemm(a[:, h, :], w_nk[h], out[:, h, :])

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor, cache) -> None:
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        H, d, dr, dv, Q, R = s.heads, s.head_dim, s.rot_dim, s.value_dim, s.q_rank, s.kv_rank
        if cache is None:
            raise ValueError("attention needs a key/value cache plane")
        if cache.k.dtype != x.dtype:
            raise ValueError(f"attention: cache holds {cache.k.dtype}, activations are {x.dtype}")
        lat = torch.empty((rows, Q + R + dr), dtype=x.dtype, device=x.device)
        ops.gemm(x, self.down, lat)
        cos, sin, _ = self.position.kernel_args()
        cq = torch.empty((rows, Q), dtype=x.dtype, device=x.device)
        ops.latent_prep(lat, cq, self.q_norm, self.kv_norm, float(s.eps), cos, sin, Q, R, dr, batch.row_pos, batch.row_seq, batch.seq_slot,
                        cache.block_table, cache.k, cache.writable)
        q = torch.empty((rows, H * (d + dr)), dtype=x.dtype, device=x.device)
        ops.gemm(cq, self.uq, q)
        qa = torch.empty((rows, H * self.key_dim), dtype=x.dtype, device=x.device)       # per head [W_uk^T q_plain | rotated part]
        self._per_head(q.view(rows, H, d + dr)[:, :, :d], self.uk_kn, self.uk_nk, qa.view(rows, H, self.key_dim)[:, :, :R])
        ops.latent_q_rot(q, qa, H, d, dr, cos, sin, batch.row_pos)
        mixed = torch.empty((rows, H * R), dtype=x.dtype, device=x.device)               # per head sum_j p_j c_j
        splits, scratch = self.key_splits(batch)
        ops.attention(qa, mixed, cache.k, cache.v, cache.block_table, batch.seq_slot, batch.seq_q_start, batch.seq_q_len, batch.seq_kv_len,
                      batch.nseq, batch.max_q_len, H, 1, self.key_dim, float(s.scale), int(s.window), splits, scratch, value_dim=R,
                      chunk=int(s.chunk))
        ctx = torch.empty((rows, H * dv), dtype=x.dtype, device=x.device)
        self._per_head(mixed.view(rows, H, R), self.uv_kn, self.uv_nk, ctx.view(rows, H, dv))
        ops.gemm(ctx, self.o, out)
