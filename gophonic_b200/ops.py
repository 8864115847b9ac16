"""Python face of the sm_100a kernel library.

Each function checks its tensors (device, dtype, layout, sizes), passes raw pointers and the
current torch CUDA stream to the C entry point, and raises ``KernelError`` with the library's own
message if the kernel refuses the call.  Nothing here computes: there is no CPU path and no
torch fallback.  Importing this module builds the library if needed and fails if that fails.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, byref, c_float, c_int, c_int64, c_uint64, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

PAGE = 64  # tokens per cache page; the kernels' GB_PAGE

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


_lib = _build.load()


def library_file() -> str:
    return _lib._name


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_device_index = []


def use_device(index: int) -> None:
    """Make CUDA device ``index`` the current one and the one whose stream the kernels are launched
    on.  The library serves one GPU at a time; a model opened on another device moves it there."""
    torch.cuda.set_device(index)
    _device_index[:] = [index]


def _stream() -> c_void_p:
    """torch's current CUDA stream of the library's device, as a raw handle (asked anew at every
    call: a graph capture runs on a stream of its own)."""
    if _raw_stream is not None:
        if not _device_index:
            _device_index.append(torch.cuda.current_device())
        return c_void_p(_raw_stream(_device_index[0]))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


launches = 0  # kernels launched through this module since import (a call that launches two counts two)


def _check(rc: int, kernels: int = 1) -> None:
    global launches
    if rc != 0:
        raise KernelError(_lib.gb_last_error().decode("utf-8", "replace"))
    launches += kernels


def _need(t: torch.Tensor, name: str, dtype=None, dim=None, contiguous=True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; kernels run on CUDA tensors only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: dtype {t.dtype}, want {dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name}: {t.dim()} dimensions, want {dim}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: tensor is not contiguous")


# ---- embedding ---------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, stats: Optional[torch.Tensor] = None,
                 next_weight: Optional[torch.Tensor] = None, next_x: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """out[r, :] = float32(table[ids[r], :]) * scale (one float32 multiplication; 1 changes no bit).  With ``stats`` (float32 [>= rows, capacity]) the sum of
    squares of row r is left in stats[r, 0]: one partial sum a row.  With ``next_weight`` (float32
    [hidden]) and ``next_x`` (bfloat16 [rows, hidden]) also next_x = bf16(out * next_weight): the
    output of an RMSNorm with that weight but for each row's factor."""
    _need(table, "embed table", dim=2)
    _need(ids, "ids", torch.int32, 1)
    _need(out, "embed out", torch.float32, 2)
    rows, hidden = out.shape
    if ids.numel() != rows or table.shape[1] != hidden:
        raise KernelError(f"embed_gather: {ids.numel()} ids, table {tuple(table.shape)}, out {tuple(out.shape)}")
    stride = 0
    if stats is not None:
        _need(stats, "row statistics", torch.float32, 2)
        if stats.shape[0] < rows:
            raise KernelError(f"embed_gather: statistics for {stats.shape[0]} rows, {rows} rows")
        stride = stats.stride(0)
    ldxn = _check_next(next_weight, next_x, rows, hidden, "embed_gather")
    _check(_lib.gb_embed_gather_scaled(_ptr(table), _code(table.dtype), _ptr(ids), c_int(rows), c_int(hidden),
                                c_int(table.shape[0]), _ptr(out), _ptr(stats), c_int64(stride), _ptr(next_weight), _ptr(next_x),
                                c_int64(ldxn), c_float(scale), _stream()))


def _check_next(next_weight, next_x, rows: int, width: int, who: str) -> int:
    if next_weight is None:
        return 0
    _need(next_weight, "next norm weight", torch.float32, 1)
    if next_x is None:
        raise KernelError(f"{who}: a norm weight is given without a tensor for the rows it scales")
    _need(next_x, "prescaled rows", torch.bfloat16, 2, contiguous=False)
    if next_weight.numel() != width or next_x.shape != (rows, width) or next_x.stride(1) != 1:
        raise KernelError(f"{who}: norm weight of {next_weight.numel()}, prescaled rows {tuple(next_x.shape)} for {rows} x {width}")
    return next_x.stride(0)


# ---- cache pages, seeded fill ------------------------------------------------------------
def block_table_set(table: torch.Tensor, triples: torch.Tensor, n: int) -> None:
    """table[slot, logical page] = physical page for the first ``n`` (slot, logical, physical)
    triples of the int32 tensor ``triples``."""
    _need(table, "block table", torch.int32, 2)
    _need(triples, "page triples", torch.int32, 1)
    if triples.numel() < 3 * n:
        raise KernelError(f"block_table_set: {triples.numel()} integers for {n} triples")
    _check(_lib.gb_block_table_set(_ptr(table), c_int(table.stride(0)), c_int(table.shape[0]), _ptr(triples), c_int(n), _stream()))


def zero_pages(planes: torch.Tensor, triples: torch.Tensor, n: int) -> None:
    """Clear, in every plane of ``planes`` [planes, pages, ...], the pages named by the third entry
    of the first ``n`` triples."""
    _need(planes, "cache planes", dim=None)
    _need(triples, "page triples", torch.int32, 1)
    if planes.dim() < 3 or triples.numel() < 3 * n:
        raise KernelError(f"zero_pages: planes {tuple(planes.shape)}, {triples.numel()} integers for {n} triples")
    es = planes.element_size()
    _check(_lib.gb_zero_pages(_ptr(planes), c_int64(planes.stride(0) * es), c_int(planes.shape[0]), c_int64(planes.stride(1) * es),
                              c_int(planes.shape[1]), _ptr(triples), c_int(n), _stream()))


def random_fill(out: torch.Tensor, key: int, c: float, mean: float) -> None:
    """The seeded fill of ``weights.random_init``: out[i] = (sum of eight 16-bit fields of two
    splitmix64 words of (key, i) - 262140) * c + mean, the same bits the numpy writer computes."""
    _need(out, "fill target")
    _check(_lib.gb_random_fill(_ptr(out), _code(out.dtype), c_int64(out.numel()), c_uint64(key & 0xFFFFFFFFFFFFFFFF), c_float(c),
                               c_float(mean), _stream()))


# ---- norm --------------------------------------------------------------------------------
def gather_tokens(ids: torch.Tensor, source: torch.Tensor) -> None:
    """ids[i] = source[ids[i]] in place (both int32 on the device)."""
    _need(ids, "ids", torch.int32, 1)
    _need(source, "token source", torch.int32, 1)
    _check(_lib.gb_gather_tokens(_ptr(ids), _ptr(source), c_int(ids.numel()), c_int(source.numel()), _stream()))


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """h += delta (if given, in place, unless ``rows`` selects); out = rmsnorm(h) * weight."""
    _need(h, "residual", torch.float32, 2)
    _need(weight, "norm weight", torch.float32, 1)
    _need(out, "norm out", dim=2)
    n = h.shape[1]
    if weight.numel() != n or out.shape[1] != n:
        raise KernelError(f"add_rmsnorm: residual width {n}, weight {weight.numel()}, out {tuple(out.shape)}")
    if delta is not None:
        _need(delta, "delta", torch.float32, 2)
        if delta.shape != h.shape:
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs residual {tuple(h.shape)}")
    if rows is not None:
        _need(rows, "row index", torch.int32, 1)
        out_rows = rows.numel()
    else:
        out_rows = h.shape[0]
    if out.shape[0] != out_rows:
        raise KernelError(f"add_rmsnorm: out has {out.shape[0]} rows, want {out_rows}")
    _check(_lib.gb_add_rmsnorm(_ptr(h), _ptr(delta), _ptr(weight), c_float(eps), c_int(n), _ptr(out),
                               _code(out.dtype), _ptr(rows), c_int(out_rows), _stream()))


def add_rows(h: torch.Tensor, delta: torch.Tensor) -> None:
    _need(h, "residual", torch.float32, 2)
    _need(delta, "delta", torch.float32, 2)
    if delta.shape != h.shape:
        raise KernelError(f"add_rows: {tuple(delta.shape)} vs {tuple(h.shape)}")
    _check(_lib.gb_add_rows(_ptr(h), _ptr(delta), c_int(h.shape[0]), c_int(h.shape[1]), _stream()))


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    """out[r] += bias, float32 rows: the bias of a projection whose product left float32."""
    _need(out, "rows", torch.float32, 2)
    _need(bias, "bias", torch.float32, 1)
    if bias.numel() != out.shape[1]:
        raise KernelError(f"add_bias: a bias of {bias.numel()} for rows of {out.shape[1]}")
    _check(_lib.gb_add_bias(_ptr(out), _ptr(bias), c_int(out.shape[0]), c_int(out.shape[1]), _stream()))


def concat_cast(h: torch.Tensor, delta: Optional[torch.Tensor], side: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = [h[r] (+ delta[r]) | side[r]] in ``out``'s dtype: two float32 rows side by side as one product's input."""
    _need(h, "residual", torch.float32, 2)
    _need(side, "second rows", torch.float32, 2)
    _need(out, "joined rows", dim=2)
    if delta is not None:
        _need(delta, "delta", torch.float32, 2)
    rows, n = h.shape
    if side.shape != h.shape or out.shape != (rows, 2 * n) or (delta is not None and delta.shape != h.shape):
        raise KernelError(f"concat_cast: {tuple(h.shape)} and {tuple(side.shape)} into {tuple(out.shape)}")
    _check(_lib.gb_concat_cast(_ptr(h), _ptr(delta), _ptr(side), _ptr(out), _code(out.dtype), c_int(rows), c_int(n), _stream()))


# ---- feed-forward activation -------------------------------------------------------------
def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleave8: bool = False) -> None:
    """out[r, i] = silu(gate[r, i]) * up[r, i]; gate and up are the two halves of ``gate_up``'s
    columns, or, with ``interleave8``, alternate in blocks of eight columns."""
    _need(gate_up, "gate_up", dim=2)
    _need(out, "swiglu out", gate_up.dtype, 2)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2):
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
    _check(_lib.gb_swiglu(_ptr(gate_up), _ptr(out), _code(out.dtype), c_int(rows), c_int(two_i // 2),
                          c_int(1 if interleave8 else 0), _stream()))


def gemm_add_accepts(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether ``gemm_add`` takes this product: a prompt-sized bfloat16 product into a float32 ``out``."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.float32 and a.dim() == 2
            and a.shape[0] >= TC5_PAIR_MIN_ROWS and w.is_contiguous() and tc5_accepts(a, w, out)
            and out.stride(0) % 4 == 0 and out.data_ptr() % 16 == 0)


def gemm_add(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """out += a @ w^T (+ ``bias``, a float32 vector over the columns) in the epilogue of the tiled tcgen05 kernel
    (``out`` float32: the residual stream); the sum per element is out + (product + bias), all float32."""
    _need(a, "gemm a", torch.bfloat16, 2, contiguous=False)
    _need(w, "gemm w", torch.bfloat16, 2)
    _need(out, "gemm out", torch.float32, 2, contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or out.stride(1) != 1 or not gemm_add_accepts(a, w, out):
        raise KernelError(f"gemm_add: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32, 1)
        if bias.numel() != N:
            raise KernelError(f"gemm_add: a bias of {bias.numel()} for {N} columns")
        _check(_lib.gb_gemm_tc5_pair_bias(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                          c_int64(a.stride(0)), c_int64(out.stride(0)), c_int(1), _ptr(bias), _stream()))
        return
    _check(_lib.gb_gemm_tc5_pair_add(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_int64(a.stride(0)),
                                     c_int64(out.stride(0)), _stream()))


def gemm_swiglu_accepts(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_swiglu`` takes this product: bfloat16 operands the tensor-core kernels accept,
    gate/up rows interleaved in blocks of eight (every one of those kernels has the fused epilogue)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[0] % 16 == 0 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous())


def gemm_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, algo: str = "auto") -> None:
    """out[M, N/2] = silu(a Wg^T) * (a Wu^T) in one kernel, the one ``gemm`` would pick for a
    product of these sizes; ``w`` [N, K] holds gate and up rows interleaved in blocks of eight."""
    _need(a, "gemm a", torch.bfloat16, 2, contiguous=False)
    _need(w, "gemm w", torch.bfloat16, 2)
    _need(out, "gemm out", dim=2, contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2) or out.stride(1) != 1 or not gemm_swiglu_accepts(a, w):
        raise KernelError(f"gemm_swiglu: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if algo == "auto":
        algo = gemm_algo(M, N, K)
    if algo == "tc5_pair":
        _check(_lib.gb_gemm_tc5_pair_swiglu(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                            c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5":
        _check(_lib.gb_gemm_tc5_swiglu(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                       c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5_decode":
        _tc5_decode(a, w, out, 1)
    elif algo == "skinny":
        _check(_lib.gb_gemm_skinny_swiglu(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                          c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    else:
        raise KernelError(f"gemm_swiglu: unknown algorithm '{algo}'")


# ---- few-row products with the residual's row-wise work folded in ------------------------
FOLD_ROWS = int(_lib.gb_dispatch_constant(c_int(5)))   # the folded products take up to this many rows


def fold_capacity(width: int) -> int:
    """Partial sums a row that a statistics buffer must have room for when ``gemm_residual`` writes a
    residual ``width`` wide: one per 16 columns (the kernel for more than 8 rows leaves one per 128)."""
    return (width + 15) // 16


def _skinny_operands_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= FOLD_ROWS
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.is_contiguous() and w.data_ptr() % 16 == 0)


def gemm_scaled_accepts(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_scaled`` takes this product: up to 64 bfloat16 rows against bfloat16 weights
    whose rows are 16-byte aligned."""
    return _skinny_operands_ok(x, w)


def gemm_scaled(x: torch.Tensor, eps: float, stats: torch.Tensor, stats_count: int, w: torch.Tensor, out: torch.Tensor,
                swiglu: bool = False) -> str:
    """out[r] = rs[r] * (x[r] @ w^T) with rs[r] = 1 / sqrt(sum_r / K + eps), sum_r the sum of the
    ``stats_count`` partial sums stats[r, :stats_count]: the product of RMSNorm rows whose factor was
    left out when ``x = bf16(h * norm_weight)`` was made (by ``gemm_residual`` or ``embed_gather``).
    With ``swiglu``, ``w`` holds gate and up rows interleaved in blocks of eight and
    out[M, N / 2] = silu(gate) * up.  Returns the kernel's name."""
    _need(x, "prescaled rows", torch.bfloat16, 2, contiguous=False)
    _need(stats, "row statistics", torch.float32, 2)
    _need(w, "gemm w", torch.bfloat16, 2)
    _need(out, "gemm out", dim=2, contiguous=False)
    M, K = x.shape
    N = w.shape[0]
    if (not gemm_scaled_accepts(x, w) or w.shape[1] != K or out.stride(1) != 1
            or out.shape != (M, N // 2 if swiglu else N) or stats.shape[0] < M or not 0 < stats_count <= stats.shape[1]):
        raise KernelError(f"gemm_scaled: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, "
                          f"{stats_count} partial sums in {tuple(stats.shape)}")
    if _ALGO_NAMES[int(_lib.gb_gemm_scaled_algo(c_int(M), c_int(N), c_int(K), c_int(_sms())))] == "skinny":
        _check(_lib.gb_gemm_skinny_scaled(_ptr(x), c_int64(x.stride(0)), c_float(eps), _ptr(stats), c_int(stats_count),
                                          c_int64(stats.stride(0)), _ptr(w), _ptr(out), _code(out.dtype), c_int64(out.stride(0)),
                                          c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), _stream()))
        return "skinny"
    splits = int(_lib.gb_gemm_tc5_decode_splits(c_int(M), c_int(N), c_int(K), c_int(_sms())))
    _check(_lib.gb_gemm_tc5_decode_scaled(_ptr(x), c_int64(x.stride(0)), c_float(eps), _ptr(stats), c_int(stats_count),
                                          c_int64(stats.stride(0)), _ptr(w), _ptr(out), _code(out.dtype), c_int64(out.stride(0)),
                                          c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), c_int(splits), _stream()))
    return "tc5_decode"


def gemm_residual_accepts(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor) -> bool:
    return _skinny_operands_ok(x, w) and h.dtype == torch.float32 and h.stride(1) == 1


def gemm_residual(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, stats: torch.Tensor,
                  next_weight: Optional[torch.Tensor] = None, next_x: Optional[torch.Tensor] = None, behind: str = "") -> int:
    """h += x @ w^T in place (``h`` float32: the residual stream; one float32 addition per element,
    as a separate add gives) and stats[row, c] = the sum of squares of the new values of the row
    in the c-th block of columns (16 wide up to 8 rows, 128 wide above).  With ``next_weight`` also next_x = bf16(h * next_weight), the rows
    ``gemm_scaled`` takes.  ``stats`` needs ``fold_capacity(N)`` columns.  ``behind``: the kernel
    that made ``x`` (what ``gemm_scaled`` returned), if the caller knows it; a few-row kernel behind
    the tcgen05 decode kernel is launched as an ordinary kernel.  Returns the number of partial sums
    a row."""
    _need(x, "gemm a", torch.bfloat16, 2, contiguous=False)
    _need(w, "gemm w", torch.bfloat16, 2)
    _need(h, "residual", torch.float32, 2, contiguous=False)
    _need(stats, "row statistics", torch.float32, 2)
    M, K = x.shape
    N = w.shape[0]
    count = fold_capacity(N)
    if not gemm_residual_accepts(x, w, h) or w.shape[1] != K or h.shape != (M, N) or stats.shape[0] < M or stats.shape[1] < count:
        raise KernelError(f"gemm_residual: x {tuple(x.shape)}, w {tuple(w.shape)}, h {tuple(h.shape)}, statistics {tuple(stats.shape)}")
    ldxn = _check_next(next_weight, next_x, M, N, "gemm_residual")
    if gemm_algo(M, N, K) == "skinny":
        _check(_lib.gb_gemm_skinny_residual(_ptr(x), c_int64(x.stride(0)), _ptr(w), _ptr(h), c_int64(h.stride(0)), _ptr(stats),
                                            c_int64(stats.stride(0)), _ptr(next_weight), _ptr(next_x), c_int64(ldxn),
                                            c_int(M), c_int(N), c_int(K), c_int(1 if behind == "tc5_decode" else 0), _stream()))
        return count
    splits = int(_lib.gb_gemm_tc5_decode_splits(c_int(M), c_int(N), c_int(K), c_int(_sms())))
    made = c_int(0)
    _check(_lib.gb_gemm_tc5_decode_residual(_ptr(x), c_int64(x.stride(0)), _ptr(w), _ptr(h), c_int64(h.stride(0)), _ptr(stats),
                                            c_int64(stats.stride(0)), byref(made), _ptr(next_weight), _ptr(next_x), c_int64(ldxn),
                                            c_int(M), c_int(N), c_int(K), c_int(splits), _stream()))
    return made.value


# ---- matrix products ---------------------------------------------------------------------
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T with fp32 multiply-add on the CUDA cores (any dtypes)."""
    _need(a, "gemm a", dim=2, contiguous=False)
    _need(w, "gemm w", dim=2)
    _need(out, "gemm out", dim=2, contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check(_lib.gb_gemm_simt(_ptr(a), _code(a.dtype), _ptr(w), _code(w.dtype), _ptr(out), _code(out.dtype),
                             c_int(M), c_int(N), c_int(K), c_int64(a.stride(0)), c_int64(w.stride(0)),
                             c_int64(out.stride(0)), _stream()))


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, algo: str = "auto", bias: Optional[torch.Tensor] = None) -> str:
    """out = a @ w^T, choosing the kernel by operand types and sizes.  Returns the kernel's name.
    ``bias`` (a float32 vector over the columns, for a float32 ``out``) is added to the float32 sums: in the
    epilogue of the paired tcgen05 kernel and of the few-row kernel, by a row-wise kernel behind every other one.

    bfloat16 activations with bfloat16 weights go to the tensor-core kernels (``gemm_algo``): up to
    8 rows the fragment-streaming kernel, up to 64 rows (128 or 256 for narrow outputs) the tcgen05
    decode kernel, otherwise the tiled tcgen05 kernel and from 192 rows the one that pairs two SMs
    on a tile.  Everything else,
    and operands whose rows are not 16-byte aligned, goes to the fp32 CUDA-core kernel.  float32
    operands never touch a tensor core.
    """
    _need(a, "gemm a", dim=2, contiguous=False)
    _need(w, "gemm w", dim=2)
    _need(out, "gemm out", dim=2, contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"gemm: output dtype {out.dtype}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32, 1)
        if bias.numel() != N or out.dtype != torch.float32:
            raise KernelError(f"gemm: a bias of {bias.numel()} for {N} columns of {out.dtype}")
        fused = ""
        if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and a.stride(0) % 8 == 0
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous()):
            fused = gemm_algo(M, N, K) if algo == "auto" else algo
        if fused == "tc5_pair":
            _check(_lib.gb_gemm_tc5_pair_bias(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                              c_int64(a.stride(0)), c_int64(out.stride(0)), c_int(0), _ptr(bias), _stream()))
            return fused
        if fused == "skinny":
            _check(_lib.gb_gemm_skinny_bias(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                            c_int64(a.stride(0)), c_int64(out.stride(0)), _ptr(bias), _stream()))
            return fused
        name = gemm(a, w, out, algo)
        add_bias(out, bias)
        return name
    if algo == "simt" or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        gemm_simt(a, w, out)
        return "simt"
    aligned = (K % 8 == 0 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
               and a.stride(1) == 1 and w.is_contiguous())
    if not aligned:
        gemm_simt(a, w, out)
        return "simt"
    if algo == "auto":
        algo = gemm_algo(M, N, K)
    if algo == "skinny":
        _check(_lib.gb_gemm_skinny(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                   c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5":
        _check(_lib.gb_gemm_tc5(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5_pair":
        _check(_lib.gb_gemm_tc5_pair(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                     c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5_decode":
        _tc5_decode(a, w, out, 0)
    elif algo == "simt":
        gemm_simt(a, w, out)
    else:
        raise KernelError(f"gemm: unknown algorithm '{algo}'")
    return algo


_ALGO_NAMES = ("simt", "skinny", "tc5", "tc5_pair", "tc5_decode")


def gemm_algo(M: int, N: int, K: int) -> str:
    """The tensor-core kernel ``gemm`` picks for aligned bfloat16 operands of these sizes: up to 8 rows
    the fragment-streaming kernel, up to 64 rows (128 or 256 for narrow outputs) the tcgen05 decode
    kernel, otherwise the tiled tcgen05 kernel and from 192 rows the one that pairs two SMs on a
    tile.  The rule lives in the library (``gb_gemm_algo``), which also applies it when it
    issues a whole layer itself."""
    return _ALGO_NAMES[int(_lib.gb_gemm_algo(c_int(M), c_int(N), c_int(K), c_int(_sms())))]


# the rule's thresholds, as the library holds them: rows up to which the fragment-streaming kernel
# is used, rows up to which the tcgen05 decode kernel takes a product, rows from which two SMs are
# paired on a tile, and the output width from which the decode kernel takes every row count
SKINNY_MAX_ROWS, TC5_DECODE_MAX_ROWS, TC5_PAIR_MIN_ROWS, WIDE_OUTPUT, TC5_ATTENTION_MIN_ROWS = (
    int(_lib.gb_dispatch_constant(c_int(i))) for i in range(5))

_sm_count = {}


def _sms() -> int:
    """SMs of the library's device."""
    dev = _device_index[0] if _device_index else torch.cuda.current_device()
    if dev not in _sm_count:
        _sm_count[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_count[dev]


def _tc5_decode(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int) -> None:
    M, K = a.shape
    N = w.shape[0]
    splits = int(_lib.gb_gemm_tc5_decode_splits(c_int(M), c_int(N), c_int(K), c_int(_sms())))
    _check(_lib.gb_gemm_tc5_decode(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                   c_int64(a.stride(0)), c_int64(out.stride(0)), c_int(epi), c_int(splits), _stream()))


def tc5_accepts(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes this product (TMA wants 16-byte rows; edges are free)."""
    K = a.shape[1]
    return K % 8 == 0 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def is_checked_build() -> bool:
    """Whether the loaded library was compiled with bounds-checked indices (GOPHONIC_B200_CHECKED=1)."""
    return bool(_lib.gb_is_checked())


_CHECK_NAMES = {1: "a token id outside the vocabulary", 2: "a position outside the token source", 3: "a cache slot outside the block table",
                4: "a position beyond the pages of a block-table row", 5: "a block-table entry outside the cache plane",
                6: "a position beyond the rotation tables", 7: "a sequence length that does not fit", 8: "a page triple outside the table or plane"}


def checked_status():
    """None, or (where, what, value, bound, count) for the first index a kernel of the checked build
    found out of bounds since the last call (the access was skipped or redirected, nothing faulted).
    Always None in the ordinary build, whose kernels carry no checks.  Synchronises."""
    out = (c_int * 4)()
    for name in ("rows", "cache", "attention_simt", "attention_mma", "attention_tc5", "linear_state", "delta_state", "attention_sigmoid", "hyper", "postnorm", "attention_latent"):
        code = int(getattr(_lib, "gb_checked_status_" + name)(out))
        if code or out[3]:
            return name, _CHECK_NAMES.get(code, f"code {code}"), out[1], out[2], out[3]
    return None


def tc5_status() -> int:
    """0, or which role of a tcgen05 kernel gave up waiting on a barrier since the last call."""
    code = 0
    for name in ("gb_gemm_tc5_status", "gb_gemm_tc5_decode_status", "gb_attention_tc5_status"):
        code = code or int(getattr(_lib, name)())
    return code


# ---- attention ---------------------------------------------------------------------------
class _QkRopeParams(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("row_stride", c_int64), ("q_w", c_void_p), ("k_w", c_void_p), ("eps", c_float),
        ("cos_t", c_void_p), ("sin_t", c_void_p), ("rot", c_int), ("table_positions", c_int),
        ("row_pos", c_void_p), ("row_seq", c_void_p), ("seq_slot", c_void_p), ("block_table", c_void_p),
        ("bt_stride", c_int), ("k_plane", c_void_p), ("v_plane", c_void_p),
        ("write_kv", c_int), ("rows", c_int), ("heads", c_int), ("kv_heads", c_int), ("d", c_int),
        ("pages", c_int), ("max_slots", c_int),
        ("q_b", c_void_p), ("k_b", c_void_p), ("v_b", c_void_p), ("pairs", c_int), ("dv", c_int), ("span", c_int), ("v_share", c_int),
    ]


def _rope_params(qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                 q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                 cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                 row_pos: torch.Tensor, row_seq: torch.Tensor, seq_slot: torch.Tensor,
                 block_table: torch.Tensor,
                 k_plane: Optional[torch.Tensor], v_plane: Optional[torch.Tensor], write_kv: bool,
                 biases=None, pairs: bool = False, value_dim: Optional[int] = None, span: bool = False, v_share: int = 1) -> "_QkRopeParams":
    """``biases`` = (q, k, v) float32 vectors or None each, added to the heads first; ``pairs``: channels
    2j and 2j + 1 turn together instead of j and j + rotary_dim / 2; ``value_dim``: size of a value
    head if it is not ``head_dim``; ``span``: the norm runs over all heads of q together (``q_weight`` of
    heads * head_dim) and over all heads of k together, not per head; ``v_share`` > 1: that many consecutive
    key heads read one value head, so the row and the value plane hold kv_heads / v_share value heads.  With any
    of them the rows may be wider than q, k and v (what follows them is left alone)."""
    _need(qkv, "qkv", dim=2, contiguous=False)
    rows = qkv.shape[0]
    dv = head_dim if value_dim is None else int(value_dim)
    v_share = max(1, int(v_share))
    if kv_heads % v_share:
        raise KernelError(f"qk_norm_rope: {kv_heads} key heads share value heads by {v_share}")
    v_heads = kv_heads // v_share
    general = biases is not None or pairs or dv != head_dim or span or v_share > 1
    used = (heads + kv_heads) * head_dim + v_heads * dv
    if qkv.stride(1) != 1 or (qkv.shape[1] < used if general else (qkv.shape[1] != used or not qkv.is_contiguous())):
        raise KernelError(f"qk_norm_rope: qkv {tuple(qkv.shape)} for {heads}+{kv_heads} heads of {head_dim} and {kv_heads} of {dv}")
    q_b, k_b, v_b = biases if biases is not None else (None, None, None)
    for t, nm, n in ((q_b, "q bias", heads * head_dim), (k_b, "k bias", kv_heads * head_dim), (v_b, "v bias", v_heads * dv)):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.numel() != n:
                raise KernelError(f"qk_norm_rope: {nm} has {t.numel()} elements, want {n}")
    for t, nm, n in ((q_weight, "q norm", heads * head_dim if span else head_dim), (k_weight, "k norm", kv_heads * head_dim if span else head_dim)):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.numel() != n:
                raise KernelError(f"qk_norm_rope: {nm} weight has {t.numel()} elements, want {n}")
    table_positions = 0
    if rotary_dim > 0:
        _need(cos, "rope cos", torch.float32, 2)
        _need(sin, "rope sin", torch.float32, 2)
        if cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"qk_norm_rope: angle tables {tuple(cos.shape)} for rotary width {rotary_dim}")
        table_positions = cos.shape[0]
    for t, nm in ((row_pos, "row_pos"), (row_seq, "row_seq"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if write_kv:
        for t, nm, n, nh in ((k_plane, "key plane", head_dim, kv_heads), (v_plane, "value plane", dv, v_heads)):
            _need(t, nm, qkv.dtype, 4)
            if t.shape[1] != nh or t.shape[2] != PAGE or t.shape[3] != n:
                raise KernelError(f"qk_norm_rope: {nm} {tuple(t.shape)} for {nh} kv heads of {n}")
    p = _QkRopeParams(qkv.data_ptr(), qkv.stride(0), 0 if q_weight is None else q_weight.data_ptr(),
                      0 if k_weight is None else k_weight.data_ptr(), eps,
                      0 if cos is None else cos.data_ptr(), 0 if sin is None else sin.data_ptr(), rotary_dim,
                      table_positions, row_pos.data_ptr(), row_seq.data_ptr(), seq_slot.data_ptr(),
                      block_table.data_ptr(), block_table.stride(0),
                      0 if k_plane is None else k_plane.data_ptr(), 0 if v_plane is None else v_plane.data_ptr(),
                      1 if write_kv else 0, rows, heads, kv_heads, head_dim,
                      0 if k_plane is None else k_plane.shape[0], block_table.shape[0],
                      0 if q_b is None else q_b.data_ptr(), 0 if k_b is None else k_b.data_ptr(),
                      0 if v_b is None else v_b.data_ptr(), 1 if pairs else 0, dv, 1 if span else 0, v_share)
    return p


def qk_norm_rope_kv_write(qkv: torch.Tensor, *args, **kwargs) -> None:
    """Biases (optional), per-head RMSNorm of q and k (optional), rotary embedding of both, q in place,
    k and v into the cache: (qkv, heads, kv_heads, head_dim, q_weight, k_weight, eps, cos, sin,
    rotary_dim, row_pos, row_seq, seq_slot, block_table, k_plane, v_plane, write_kv) and the keywords
    of ``_rope_params``."""
    p = _rope_params(qkv, *args, **kwargs)
    _check(_lib.gb_qk_norm_rope_kv_write_x(byref(p), _code(qkv.dtype), _stream()))


class _AttnParams(Structure):
    _fields_ = [
        ("q", c_void_p), ("q_row_stride", c_int64), ("out", c_void_p), ("out_row_stride", c_int64),
        ("k_plane", c_void_p), ("v_plane", c_void_p), ("block_table", c_void_p), ("bt_stride", c_int),
        ("seq_slot", c_void_p), ("seq_q_start", c_void_p), ("seq_q_len", c_void_p),
        ("seq_kv_len", c_void_p), ("nseq", c_int), ("heads", c_int), ("kv_heads", c_int), ("d", c_int),
        ("max_q_len", c_int), ("scale", c_float), ("window", c_int), ("num_splits", c_int), ("scratch", c_void_p),
        ("pages", c_int), ("max_slots", c_int), ("dv", c_int), ("keep_first", c_int), ("sink", c_int), ("sinks", c_void_p),
        ("chunk", c_int), ("v_share", c_int), ("v_row_stride", c_int64),
    ]


def attention_scratch_floats(nseq: int, heads: int, head_dim: int, num_splits: int) -> int:
    return nseq * heads * num_splits * (head_dim + 2)


def _attn_params(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                 block_table: torch.Tensor, seq_slot: torch.Tensor, seq_q_start: torch.Tensor,
                 seq_q_len: torch.Tensor, seq_kv_len: torch.Tensor, nseq: int, max_q_len: int,
                 heads: int, kv_heads: int, head_dim: int, scale: float, window: int,
                 num_splits: int, scratch: Optional[torch.Tensor], value_dim: Optional[int] = None, keep_first: int = 0,
                 sink: bool = False, sinks: Optional[torch.Tensor] = None, chunk: int = 0, v_share: int = 1) -> "_AttnParams":
    """``value_dim``: size of a value head if it is not ``head_dim``; ``keep_first``: with a window, keys
    at positions below it stay visible; ``sink``: one more unit in the softmax denominator; ``sinks``
    (float32 [heads]): head h's denominator holds exp(sinks[h]) instead of that unit; ``chunk`` > 0: row i
    sees key j <= i only if both lie in the same block of ``chunk`` positions counted from the sequence's
    start; ``v_share`` > 1: that many consecutive key heads read one value head (the value plane holds
    kv_heads / v_share heads).  The value plane may be a view whose tokens lie further apart than
    ``value_dim`` (the first channels of a wider plane, the key plane itself for instance)."""
    _need(q, "attention q", dim=2, contiguous=False)
    _need(out, "attention out", q.dtype, 2, contiguous=False)
    dv = head_dim if value_dim is None else int(value_dim)
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] < heads * head_dim or out.shape[1] < heads * dv:
        raise KernelError(f"attention: q {tuple(q.shape)}, out {tuple(out.shape)} for {heads} heads of {head_dim} / {dv}")
    if keep_first < 0:
        raise KernelError(f"attention: {keep_first} kept first tokens")
    if sinks is not None:
        _need(sinks, "sink scores", torch.float32, 1)
        if sinks.numel() != heads:
            raise KernelError(f"attention: {sinks.numel()} sink scores for {heads} heads")
    v_share = max(1, int(v_share))
    if chunk < 0 or kv_heads % v_share:
        raise KernelError(f"attention: blocks of {chunk} positions, {kv_heads} key heads sharing value heads by {v_share}")
    _need(k_plane, "key plane", q.dtype, 4)
    _need(v_plane, "value plane", q.dtype, 4, contiguous=False)
    for t, nm, n, nh in ((k_plane, "key plane", head_dim, kv_heads), (v_plane, "value plane", dv, kv_heads // v_share)):
        if t.shape[1] != nh or t.shape[2] != PAGE or t.shape[3] != n:
            raise KernelError(f"attention: {nm} {tuple(t.shape)} for {nh} kv heads of {n}")
    v_tok = v_plane.stride(2)
    if v_plane.stride(3) != 1 or v_tok < dv or v_plane.stride(1) != PAGE * v_tok or v_plane.stride(0) != v_plane.shape[1] * PAGE * v_tok:
        raise KernelError(f"attention: value plane with strides {tuple(v_plane.stride())}")
    for t, nm in ((seq_slot, "seq_slot"), (seq_q_start, "seq_q_start"), (seq_q_len, "seq_q_len"),
                  (seq_kv_len, "seq_kv_len")):
        _need(t, nm, torch.int32, 1)
        if t.numel() < nseq:
            raise KernelError(f"attention: {nm} has {t.numel()} entries for {nseq} sequences")
    _need(block_table, "block table", torch.int32, 2)
    if num_splits > 1:
        if scratch is None:
            raise KernelError("attention: key splits need scratch memory")
        _need(scratch, "attention scratch", torch.float32)
        if scratch.numel() < attention_scratch_floats(nseq, heads, dv, num_splits):
            raise KernelError("attention: scratch is too small")
    p = _AttnParams(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_plane.data_ptr(), v_plane.data_ptr(),
                    block_table.data_ptr(), block_table.stride(0), seq_slot.data_ptr(),
                    seq_q_start.data_ptr(), seq_q_len.data_ptr(), seq_kv_len.data_ptr(), nseq, heads, kv_heads,
                    head_dim, max_q_len, scale, window, num_splits, 0 if scratch is None else scratch.data_ptr(),
                    k_plane.shape[0], block_table.shape[0], 0 if dv == head_dim else dv, int(keep_first) if window > 0 else 0,
                    1 if sink or sinks is not None else 0, 0 if sinks is None else sinks.data_ptr(),
                    int(chunk), v_share, 0 if v_tok == dv else v_tok)
    return p


def attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
              block_table: torch.Tensor, seq_slot: torch.Tensor, seq_q_start: torch.Tensor,
              seq_q_len: torch.Tensor, seq_kv_len: torch.Tensor, nseq: int, max_q_len: int,
              heads: int, kv_heads: int, head_dim: int, scale: float, window: int = 0,
              num_splits: int = 1, scratch: Optional[torch.Tensor] = None, algo: str = "auto",
              value_dim: Optional[int] = None, keep_first: int = 0, sink: bool = False, sinks: Optional[torch.Tensor] = None,
              chunk: int = 0, v_share: int = 1) -> str:
    """Causal GQA over the paged cache.  q is a [rows, >= heads*head_dim] view (row stride free),
    out is [rows, heads*value_dim].  Returns the kernel's name."""
    p = _attn_params(q, out, k_plane, v_plane, block_table, seq_slot, seq_q_start, seq_q_len, seq_kv_len, nseq, max_q_len,
                     heads, kv_heads, head_dim, scale, window, num_splits, scratch, value_dim, keep_first, sink, sinks, chunk, v_share)
    if algo == "auto":   # the library's own rule (head size, rows per sequence, alignment)
        algo = ("simt", "decode_mma", "prefill_mma", "prefill_tc5", "latent_mma")[int(_lib.gb_attention_algo_x(byref(p), _code(q.dtype)))]
    nk = 2 if num_splits > 1 else 1
    if algo == "simt":
        _check(_lib.gb_attention_simt_x(byref(p), _code(q.dtype), _stream()), nk)
    elif algo == "decode_mma":
        _check(_lib.gb_attention_decode_mma_x(byref(p), _stream()), nk)
    elif algo == "prefill_mma":
        _check(_lib.gb_attention_prefill_mma_x(byref(p), _stream()))
    elif algo == "prefill_tc5":
        _check(_lib.gb_attention_prefill_tc5_x(byref(p), c_int(q.shape[0]), c_int(k_plane.shape[0]), _stream()))
    elif algo == "latent_mma":
        _check(_lib.gb_attention_latent_mma(byref(p), _stream()), nk)
    else:
        raise KernelError(f"attention: unknown algorithm '{algo}'")
    return algo


def attention_decode_rope_accepts(dtype: torch.dtype, head_dim: int, rotary_dim: int, max_q_len: int) -> bool:
    """Whether ``attention_decode_rope`` takes rows of this kind (bfloat16, one row a sequence, a head
    size the tensor-core single-token kernel takes)."""
    return dtype in (torch.float32, torch.bfloat16) and bool(_lib.gb_attention_decode_rope_accepts(_code(dtype), c_int(head_dim), c_int(rotary_dim), c_int(max_q_len)))


def attention_decode_rope(qkv: torch.Tensor, out: torch.Tensor, rope_args: tuple, attn_args: tuple) -> None:
    """``qk_norm_rope_kv_write(qkv, *rope_args)`` and ``attention(qkv[:, :heads * head_dim], out,
    *attn_args)`` for single-token rows in one kernel (plus the merge of key splits): the attention
    kernel norms and rotates its queries itself, takes the token's own key and value from the row and
    stores them in the cache.  The same bits as the two calls."""
    r = _rope_params(qkv, *rope_args)
    a = _attn_params(qkv[:, :r.heads * r.d], out, *attn_args)
    _check(_lib.gb_attention_decode_mma_rope(byref(a), byref(r), _stream()), 2 if a.num_splits > 1 else 1)


# ---- mixers with a matrix state ------------------------------------------------------------
class _LinearStateParams(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("row_stride", c_int64), ("q_off", c_int), ("k_off", c_int), ("v_off", c_int), ("q_scale", c_float),
        ("decay", c_void_p), ("decay_stride", c_int64), ("gates", c_void_p), ("gates_stride", c_int64), ("gate_bias", c_void_p),
        ("gate_cap", c_float), ("coef", c_void_p), ("state", c_void_p), ("slot_stride", c_int64), ("head_stride", c_int64),
        ("out", c_void_p), ("out_stride", c_int64), ("seq_slot", c_void_p), ("seq_q_start", c_void_p), ("seq_q_len", c_void_p),
        ("nseq", c_int), ("heads", c_int), ("d", c_int), ("dv", c_int), ("scalar_decay", c_int), ("max_slots", c_int),
        ("max_q_len", c_int),
    ]


class _HeadGateParams(Structure):
    _fields_ = [
        ("x", c_void_p), ("x_stride", c_int64), ("gate", c_void_p), ("gate_stride", c_int64), ("y", c_void_p), ("y_stride", c_int64),
        ("divisor", c_void_p), ("divisor_stride", c_int), ("weight", c_void_p), ("weight_per_head", c_int), ("normed", c_int),
        ("eps", c_float), ("gate_kind", c_int), ("rows", c_int), ("heads", c_int), ("size", c_int),
    ]


GATE_SIGMOID, GATE_SILU = 0, 1


def gla_decay(z: torch.Tensor, bias: Optional[torch.Tensor], tau: float) -> None:
    """In place: z[r, c] = sigmoid(z[r, c] + bias[c]) ** (1 / tau), float32."""
    _need(z, "decay pre-activations", torch.float32, 2)
    if bias is not None:
        _need(bias, "decay bias", torch.float32, 1)
        if bias.numel() != z.shape[1]:
            raise KernelError(f"gla_decay: bias of {bias.numel()} for rows of {z.shape[1]}")
    _check(_lib.gb_gla_decay(_ptr(z), _ptr(bias), c_int(z.shape[0]), c_int(z.shape[1]), c_float(tau), _stream()))


def state_scan(qkv: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, d: int, dv: int, q_scale: float,
               state: torch.Tensor, out: torch.Tensor, seq_slot: torch.Tensor, seq_q_start: torch.Tensor, seq_q_len: torch.Tensor,
               nseq: int, decay: Optional[torch.Tensor] = None, gates: Optional[torch.Tensor] = None,
               gate_bias: Optional[torch.Tensor] = None, gate_cap: float = 0.0, coef: Optional[torch.Tensor] = None,
               max_q_len: int = 0) -> None:
    """The matrix-state recurrence S <- diag(a) S + b k v^T, o = S^T (q * q_scale) over the rows of a step,
    token by token, for every (sequence, head); ``state`` [slots, heads, d * dv (+ d + 1)] float32 is read
    and left updated, ``out`` [rows, heads * dv] float32 receives the sums.  With ``decay`` (float32 [rows,
    heads * d]) a is a factor per key channel and b = 1.  With ``gates`` (float32 [rows, 2 * heads]: input
    then forget pre-activations), ``gate_bias``, ``gate_cap`` and ``coef`` (float32 [rows, heads, 4] scratch)
    a and b are the stabilised exponential gates of a matrix memory, the state also carries the
    normaliser and the running maximum, and coef[..., 3] receives each token's divisor.  ``max_q_len``:
    the most rows a sequence brings, if known (1: every sequence brings one token, which has a kernel
    of its own; the arithmetic per element is the same)."""
    _need(qkv, "state_scan rows", dim=2, contiguous=False)
    _need(state, "state", torch.float32, 3)
    _need(out, "state_scan out", torch.float32, 2)
    rows = qkv.shape[0]
    scalar = gates is not None
    need = d * dv + (d + 1 if scalar else 0)
    if (qkv.stride(1) != 1 or out.shape != (rows, heads * dv) or state.shape[1] != heads or state.shape[2] < need
            or max(q_off, k_off) + heads * d > qkv.shape[1] or v_off + heads * dv > qkv.shape[1]):
        raise KernelError(f"state_scan: rows {tuple(qkv.shape)}, state {tuple(state.shape)}, out {tuple(out.shape)} for "
                          f"{heads} heads of {d} x {dv}")
    for t, nm in ((seq_slot, "seq_slot"), (seq_q_start, "seq_q_start"), (seq_q_len, "seq_q_len")):
        _need(t, nm, torch.int32, 1)
        if t.numel() < nseq:
            raise KernelError(f"state_scan: {nm} has {t.numel()} entries for {nseq} sequences")
    if scalar:
        _need(gates, "gates", torch.float32, 2, contiguous=False)
        _need(coef, "gate factors", torch.float32, 3)
        if gates.shape != (rows, 2 * heads) or gates.stride(1) != 1 or coef.shape[0] < rows or coef.shape[1:] != (heads, 4):
            raise KernelError(f"state_scan: gates {tuple(gates.shape)}, factors {tuple(coef.shape)}")
        if gate_bias is not None:
            _need(gate_bias, "gate bias", torch.float32, 1)
            if gate_bias.numel() != 2 * heads:
                raise KernelError(f"state_scan: gate bias of {gate_bias.numel()} for {heads} heads")
    else:
        if decay is None:
            raise KernelError("state_scan: neither decays nor gates")
        _need(decay, "decays", torch.float32, 2, contiguous=False)
        if decay.shape != (rows, heads * d) or decay.stride(1) != 1:
            raise KernelError(f"state_scan: decays {tuple(decay.shape)} for {heads} heads of {d}")
    p = _LinearStateParams(qkv.data_ptr(), qkv.stride(0), q_off, k_off, v_off, q_scale,
                           0 if decay is None else decay.data_ptr(), 0 if decay is None else decay.stride(0),
                           0 if gates is None else gates.data_ptr(), 0 if gates is None else gates.stride(0),
                           0 if gate_bias is None else gate_bias.data_ptr(), gate_cap, 0 if coef is None else coef.data_ptr(),
                           state.data_ptr(), state.stride(0), state.stride(1), out.data_ptr(), out.stride(0),
                           seq_slot.data_ptr(), seq_q_start.data_ptr(), seq_q_len.data_ptr(), nseq, heads, d, dv,
                           1 if scalar else 0, state.shape[0], int(max_q_len))
    _check(_lib.gb_state_scan(byref(p), _code(qkv.dtype), _stream()), 2 if scalar else 1)


def head_norm_gate(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor, heads: int, size: int, gate_kind: int,
                   weight: Optional[torch.Tensor] = None, eps: Optional[float] = None, divisor: Optional[torch.Tensor] = None) -> None:
    """y[r, h] = norm(x[r, h] / divisor[r, h]) * weight * gate(g[r, h]) for heads of ``size``: the division
    only with ``divisor`` (float32 [rows, heads, 1], possibly a column of a wider tensor), the norm (x over its root mean
    square, eps under the root) only with ``eps``, the weight ([size], shared by the heads, or
    [heads * size]) only if given; the gate is sigmoid(g) or, with ``GATE_SILU``, g * sigmoid(g).
    x is float32 or the activation dtype; g and y are the activation dtype; all arithmetic float32."""
    _need(x, "head_norm_gate x", dim=2, contiguous=False)
    _need(gate, "head_norm_gate gate", y.dtype, 2, contiguous=False)
    _need(y, "head_norm_gate y", dim=2, contiguous=False)
    rows = x.shape[0]
    n = heads * size
    if (x.shape[1] < n or gate.shape != (rows, n) or y.shape != (rows, n) or x.stride(1) != 1 or gate.stride(1) != 1 or y.stride(1) != 1):
        raise KernelError(f"head_norm_gate: x {tuple(x.shape)}, gate {tuple(gate.shape)}, y {tuple(y.shape)} for {heads} heads of {size}")
    per_head = 0
    if weight is not None:
        _need(weight, "head norm weight", torch.float32, 1)
        if weight.numel() not in (size, n):
            raise KernelError(f"head_norm_gate: weight of {weight.numel()} for {heads} heads of {size}")
        per_head = 1 if weight.numel() == n and heads > 1 else 0
    dstride = 0
    if divisor is not None:
        _need(divisor, "divisor", torch.float32, 3, contiguous=False)
        dstride = divisor.stride(1)
        if divisor.shape[0] < rows or divisor.shape[1] != heads or divisor.stride(0) != heads * dstride:
            raise KernelError(f"head_norm_gate: divisor {tuple(divisor.shape)} with strides {divisor.stride()}")
    p = _HeadGateParams(x.data_ptr(), x.stride(0), gate.data_ptr(), gate.stride(0), y.data_ptr(), y.stride(0),
                        0 if divisor is None else divisor.data_ptr(), dstride, 0 if weight is None else weight.data_ptr(), per_head,
                        0 if eps is None else 1, 0.0 if eps is None else eps, gate_kind, rows, heads, size)
    _check(_lib.gb_head_norm_gate(byref(p), _code(x.dtype), _code(y.dtype), _stream()))


# ---- a whole pre-norm layer from one call ---------------------------------------------------
class PrenormLayer(Structure):
    """Sizes, constants and tensors of one pre-norm layer of attention and SwiGLU (``GbPrenormLayer``)."""
    _fields_ = [
        ("hidden", c_int), ("heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("intermediate", c_int),
        ("mixer_norm_eps", c_float), ("ffn_norm_eps", c_float), ("qk_norm_eps", c_float), ("scale", c_float),
        ("window", c_int), ("rotary_dim", c_int), ("table_positions", c_int), ("act_dtype", c_int), ("gate_up_interleaved", c_int),
        ("mixer_norm_w", c_void_p), ("ffn_norm_w", c_void_p), ("w_qkv", c_void_p), ("w_qkv_dtype", c_int), ("w_o", c_void_p),
        ("w_o_dtype", c_int), ("w_gate_up", c_void_p), ("w_gate_up_dtype", c_int), ("w_down", c_void_p), ("w_down_dtype", c_int),
        ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("cos_t", c_void_p), ("sin_t", c_void_p),
    ]


class _StepRows(Structure):
    _fields_ = [
        ("rows", c_int), ("nseq", c_int), ("max_q_len", c_int), ("row_pos", c_void_p), ("row_seq", c_void_p), ("seq_slot", c_void_p),
        ("seq_q_start", c_void_p), ("seq_q_len", c_void_p), ("seq_kv_len", c_void_p), ("num_splits", c_int), ("split_scratch", c_void_p),
        ("block_table", c_void_p), ("bt_stride", c_int), ("k_plane", c_void_p), ("v_plane", c_void_p), ("pages", c_int), ("write_kv", c_int),
        ("max_slots", c_int),
    ]


_lib.gb_prenorm_layer_workspace.restype = c_int64


def prenorm_layer_workspace(layer: PrenormLayer, rows: int) -> int:
    """Bytes of workspace ``prenorm_layer_forward`` needs for a step of ``rows`` rows."""
    return int(_lib.gb_prenorm_layer_workspace(byref(layer), c_int(rows)))


def prenorm_layer_forward(layer: PrenormLayer, batch, cache, h: torch.Tensor, delta: Optional[torch.Tensor],
                          workspace: torch.Tensor, num_splits: int = 1, split_scratch: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Issue every kernel of one pre-norm layer (norm, q/k/v product, q/k norm + rotation + cache
    write, attention, output projection, norm, gate/up product with SwiGLU, down projection) from one
    call into the library: the kernels, their order and their choice by size are those of the
    part-by-part path.  ``h`` is the float32 residual, updated in place; ``delta`` an addend it is
    still owed (added by the first norm).  Returns the addend the layer leaves owed (a view into
    ``workspace``), or None if its products added into the residual themselves."""
    _need(h, "residual", torch.float32, 2)
    _need(workspace, "layer workspace", torch.uint8, 1)
    rows = h.shape[0]
    if h.shape[1] != layer.hidden or rows != batch.rows:
        raise KernelError(f"prenorm_layer: residual {tuple(h.shape)} for {batch.rows} rows of {layer.hidden}")
    if delta is not None:
        _need(delta, "delta", torch.float32, 2)
        if delta.shape != h.shape:
            raise KernelError(f"prenorm_layer: delta {tuple(delta.shape)} vs residual {tuple(h.shape)}")
    if cache.k.dtype != (torch.bfloat16 if layer.act_dtype == BF16 else torch.float32):
        raise KernelError(f"prenorm_layer: the cache holds {cache.k.dtype}")
    step = _StepRows(rows, batch.nseq, batch.max_q_len, batch.row_pos.data_ptr(), batch.row_seq.data_ptr(), batch.seq_slot.data_ptr(),
                     batch.seq_q_start.data_ptr(), batch.seq_q_len.data_ptr(), batch.seq_kv_len.data_ptr(), num_splits,
                     0 if split_scratch is None else split_scratch.data_ptr(), cache.block_table.data_ptr(), cache.block_table.stride(0),
                     cache.k.data_ptr(), cache.v.data_ptr(), cache.k.shape[0], 1 if cache.writable else 0, cache.block_table.shape[0])
    out_ptr, n = c_void_p(0), c_int(0)
    _check(_lib.gb_prenorm_layer_forward(byref(layer), byref(step), _ptr(h), _ptr(delta), _ptr(workspace), c_int64(workspace.numel()),
                                         c_int(_sms()), byref(out_ptr), byref(n), _stream()), 0)
    global launches
    launches += n.value
    if not out_ptr.value:
        return None
    at = out_ptr.value - workspace.data_ptr()
    return workspace[at:at + 4 * rows * layer.hidden].view(torch.float32).view(rows, layer.hidden)


# ---- sampling ----------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32, 2, contiguous=False)
    _need(out, "argmax out", torch.int32, 1)
    if logits.stride(1) != 1 or out.numel() != logits.shape[0]:
        raise KernelError(f"argmax: logits {tuple(logits.shape)}, out {out.numel()}")
    rows, vocab = logits.shape
    if vocab > 16384:  # wide rows: many CTAs a row, merged by a second small kernel
        chunks = (vocab + 8191) // 8192
        scratch = torch.empty(2 * rows * chunks, dtype=torch.float32, device=logits.device)
        _check(_lib.gb_argmax_wide(_ptr(logits), c_int(rows), c_int(vocab), c_int64(logits.stride(0)), _ptr(out),
                                   _ptr(scratch), _stream()), 2)
        return
    _check(_lib.gb_argmax(_ptr(logits), c_int(rows), c_int(vocab), c_int64(logits.stride(0)), _ptr(out), _stream()))


def sample_scratch_bytes(rows: int, vocab: int) -> int:
    """Bytes of scratch with which ``sample`` spreads a row of a wide vocabulary over many CTAs."""
    _lib.gb_sample_scratch_bytes.restype = c_int64
    return int(_lib.gb_sample_scratch_bytes(c_int(rows), c_int(vocab)))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed: torch.Tensor, draw: torch.Tensor, out: torch.Tensor, opt_row: Optional[torch.Tensor] = None,
           advance: bool = False, scratch: Optional[torch.Tensor] = None) -> None:
    """One token per row: greedy where temperature <= 0, else top-k / top-p sampling with the
    counter-based draw (seed, draw).  Row i takes its options from entry ``opt_row[i]`` of the
    option tensors (entry i without ``opt_row``); with ``advance`` the kernel adds one to the draw
    counter of every row it sampled.  ``scratch`` (uint8, ``sample_scratch_bytes``) lets rows of a
    wide vocabulary be selected by many CTAs; without it one CTA scans each row."""
    _need(logits, "logits", torch.float32, 2, contiguous=False)
    rows = logits.shape[0]
    _need(temperature, "temperature", torch.float32, 1)
    _need(top_k, "top_k", torch.int32, 1)
    _need(top_p, "top_p", torch.float32, 1)
    _need(seed, "seed", torch.int64, 1)
    _need(draw, "draw", torch.int64, 1)
    _need(out, "sample out", torch.int32, 1)
    if out.numel() < rows:
        raise KernelError("sample: out is shorter than the batch")
    if opt_row is not None:
        _need(opt_row, "option rows", torch.int32, 1)
        if opt_row.numel() < rows:
            raise KernelError("sample: opt_row is shorter than the batch")
    else:
        for t in (temperature, top_k, top_p, seed, draw):
            if t.numel() < rows:
                raise KernelError("sample: a per-row option tensor is shorter than the batch")
    if logits.stride(1) != 1:
        raise KernelError("sample: logits rows are not contiguous")
    nbytes = 0
    if scratch is not None:
        _need(scratch, "sample scratch", torch.uint8, 1)
        nbytes = scratch.numel()
    want = sample_scratch_bytes(rows, logits.shape[1])
    wide = 0 < want <= nbytes
    _check(_lib.gb_sample(_ptr(logits), c_int(rows), c_int(logits.shape[1]), c_int64(logits.stride(0)), _ptr(opt_row),
                          _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(seed), _ptr(draw), _ptr(out),
                          c_int(1 if advance else 0), _ptr(scratch), c_int64(nbytes), _stream()), 3 if wide else 1)


def presence_penalty(logits: torch.Tensor, seen: torch.Tensor, seen_row: torch.Tensor, presence: torch.Tensor,
                     indexed: bool = False) -> None:
    """logits[r, v] -= presence for every token v set in bitmap row seen_row[r]; the penalty is
    presence[r], or presence[seen_row[r]] with ``indexed``."""
    _need(logits, "logits", torch.float32, 2, contiguous=False)
    _need(seen, "seen bitmap", torch.int32, 2)
    _need(seen_row, "seen row", torch.int32, 1)
    _need(presence, "presence", torch.float32, 1)
    rows, vocab = logits.shape
    if seen.shape[1] * 32 < vocab:
        raise KernelError("presence_penalty: bitmap is narrower than the vocabulary")
    _check(_lib.gb_presence_penalty(_ptr(logits), c_int(rows), c_int(vocab), c_int64(logits.stride(0)), _ptr(seen),
                                    c_int64(seen.stride(0)), _ptr(seen_row), _ptr(presence), c_int(1 if indexed else 0), _stream()))


def mark_seen(tokens: torch.Tensor, vocab: int, seen: torch.Tensor, seen_row: torch.Tensor) -> None:
    _need(tokens, "tokens", torch.int32, 1)
    _need(seen, "seen bitmap", torch.int32, 2)
    _need(seen_row, "seen row", torch.int32, 1)
    _check(_lib.gb_mark_seen(_ptr(tokens), c_int(tokens.numel()), c_int(vocab), _ptr(seen), c_int64(seen.stride(0)),
                             _ptr(seen_row), _stream()))


def f32_to_bf16(a: torch.Tensor, out: torch.Tensor) -> None:
    _need(a, "a", torch.float32)
    _need(out, "out", torch.bfloat16)
    if a.numel() != out.numel():
        raise KernelError("f32_to_bf16: sizes differ")
    _check(_lib.gb_f32_to_bf16(_ptr(a), _ptr(out), c_int64(a.numel()), _stream()))


# ---- hyper-connections -----------------------------------------------------------------------
class _HyperParams(Structure):
    _fields_ = [
        ("streams", c_void_p), ("stream_stride", c_int64), ("n_streams", c_int), ("rows", c_int), ("width", c_int),
        ("y", c_void_p), ("mix", c_void_p), ("out_coef", c_void_p), ("mult", c_float), ("in_coef", c_void_p),
        ("norm_w", c_void_p), ("eps", c_float), ("x_out", c_void_p), ("row_index", c_void_p),
    ]


def embed_streams(table: torch.Tensor, ids: torch.Tensor, streams: torch.Tensor, scale: float = 1.0) -> None:
    """streams[s, r, :] = float32(table[ids[r], :]) * scale for every stream s (``streams`` float32 [S, rows, hidden])."""
    _need(table, "embed table", dim=2)
    _need(ids, "ids", torch.int32, 1)
    _need(streams, "streams", torch.float32, 3)
    S, rows, hidden = streams.shape
    if ids.numel() != rows or table.shape[1] != hidden:
        raise KernelError(f"embed_streams: {ids.numel()} ids, table {tuple(table.shape)}, streams {tuple(streams.shape)}")
    _check(_lib.gb_embed_streams(_ptr(table), _code(table.dtype), _ptr(ids), c_int(rows), c_int(hidden), c_int(table.shape[0]), _ptr(streams),
                                 c_int64(streams.stride(0)), c_int(S), c_float(scale), _stream()))


def hyper_mix_norm(streams: torch.Tensor, y: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                   out_coef: Optional[torch.Tensor] = None, mult: float = 1.0, in_coef: Optional[torch.Tensor] = None,
                   norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, x_out: Optional[torch.Tensor] = None,
                   rows: Optional[torch.Tensor] = None) -> None:
    """The two row-wise steps around a sublayer of a residual kept in S streams (``streams`` float32
    [S, rows, width]), either or both in one pass.  With ``y`` (float32 [rows, width], a sublayer's
    output): streams[t] <- sum_s mix[s, t] streams[s] + mult * out_coef[t] * y for all t from the old
    values (``mix`` None: the identity; ``out_coef`` None: ones).  With ``x_out`` (activation dtype):
    u = sum_s in_coef[s] streams[s] (None: the plain sum) of the new values and
    x_out = u / sqrt(mean(u^2) + eps) * norm_weight.  With ``rows`` (int32 indices) x_out[i] is made
    from row rows[i] and the streams are left as they were."""
    _need(streams, "streams", torch.float32, 3)
    S, n, width = streams.shape
    for t, nm, shape in ((mix, "mix", (S, S)), (out_coef, "out coefficients", (S,)), (in_coef, "in coefficients", (S,)),
                         (norm_weight, "norm weight", (width,)), (y, "sublayer output", (n, width))):
        if t is not None:
            _need(t, nm, torch.float32)
            if tuple(t.shape) != shape:
                raise KernelError(f"hyper_mix_norm: {nm} {tuple(t.shape)}, want {shape}")
    out_rows = n
    if rows is not None:
        _need(rows, "row index", torch.int32, 1)
        out_rows = rows.numel()
    if x_out is not None:
        _need(x_out, "normed rows", dim=2)
        if x_out.shape != (out_rows, width):
            raise KernelError(f"hyper_mix_norm: normed rows {tuple(x_out.shape)}, want {(out_rows, width)}")
    p = _HyperParams(streams.data_ptr(), streams.stride(0), S, out_rows, width, 0 if y is None else y.data_ptr(),
                     0 if mix is None else mix.data_ptr(), 0 if out_coef is None else out_coef.data_ptr(), mult,
                     0 if in_coef is None else in_coef.data_ptr(), 0 if norm_weight is None else norm_weight.data_ptr(), eps,
                     0 if x_out is None else x_out.data_ptr(), 0 if rows is None else rows.data_ptr())
    _check(_lib.gb_hyper_mix_norm(byref(p), _code(x_out.dtype) if x_out is not None else F32, _stream()))


# ---- the generalized delta rule ---------------------------------------------------------------
class _DeltaStateParams(Structure):
    _fields_ = [
        ("rkv", c_void_p), ("row_stride", c_int64), ("r_off", c_int), ("k_off", c_int), ("v_off", c_int),
        ("decay", c_void_p), ("decay_stride", c_int64), ("decay_bias", c_void_p), ("decay_scale", c_float),
        ("remove", c_void_p), ("remove_stride", c_int64), ("remove_bias", c_void_p),
        ("low", c_void_p), ("low_stride", c_int64), ("w2", c_void_p), ("rank", c_int), ("key_eps", c_float), ("dots", c_void_p),
        ("state", c_void_p), ("slot_stride", c_int64), ("head_stride", c_int64), ("out", c_void_p), ("out_stride", c_int64),
        ("seq_slot", c_void_p), ("seq_q_start", c_void_p), ("seq_q_len", c_void_p),
        ("rows", c_int), ("nseq", c_int), ("heads", c_int), ("d", c_int), ("dv", c_int), ("max_slots", c_int), ("max_q_len", c_int),
    ]


DELTA_FUSED_MAX_RANK = int(_lib.gb_delta_fused_max_rank())   # largest rank of the decay's projection a single-token step folds in


def delta_scan(rkv: torch.Tensor, r_off: int, k_off: int, v_off: int, heads: int, d: int, dv: int, decay: Optional[torch.Tensor],
               decay_bias: Optional[torch.Tensor], decay_scale: float, remove: torch.Tensor, remove_bias: Optional[torch.Tensor],
               key_eps: float, state: torch.Tensor, out: torch.Tensor, seq_slot: torch.Tensor, seq_q_start: torch.Tensor,
               seq_q_len: torch.Tensor, nseq: int, max_q_len: int = 0, low: Optional[torch.Tensor] = None,
               w2: Optional[torch.Tensor] = None, prepare: bool = False) -> None:
    """The generalized delta rule over the rows of a step, token by token, for every (sequence, head):
    S <- diag(w) S - (a u)(u^T S) + k v^T from the old S, o = S^T r, with u the key over its length
    (``key_eps`` under the root).  ``decay`` and ``remove`` (float32 [rows, heads * d], row strides free) hold
    pre-activations: w = exp(-decay_scale * sigmoid(decay + decay_bias)), a = sigmoid(remove + remove_bias); a
    step of rows of more than one token overwrites both.  ``state`` [slots, heads, d * dv] float32 is read and
    left updated, ``out`` [rows, heads * dv] float32 receives the sums.  ``max_q_len`` 1: every sequence brings
    one token, which has a kernel of its own; it may be given ``low`` (float32 [rows, rank]) and ``w2``
    ([heads * d, rank]) instead of ``decay`` and then forms the decay's pre-activation w2 tanh(low) and
    everything else of the token itself, in one kernel.  ``prepare`` asks a single-token step with ``decay`` for
    the preparation kernel ahead of a lean recurrence kernel (worth it from a few dozen sequences on)."""
    _need(rkv, "delta_scan rows", dim=2, contiguous=False)
    _need(state, "state", torch.float32, 3)
    _need(out, "delta_scan out", torch.float32, 2)
    rows = rkv.shape[0]
    if (rkv.stride(1) != 1 or out.shape != (rows, heads * dv) or state.shape[1] != heads or state.shape[2] < d * dv
            or max(r_off, k_off) + heads * d > rkv.shape[1] or v_off + heads * dv > rkv.shape[1]):
        raise KernelError(f"delta_scan: rows {tuple(rkv.shape)}, state {tuple(state.shape)}, out {tuple(out.shape)} for "
                          f"{heads} heads of {d} x {dv}")
    for t, nm in ((decay, "decay pre-activations"), (remove, "removal pre-activations")):
        if t is None and nm.startswith("decay") and low is not None:
            continue
        if t is None:
            raise KernelError(f"delta_scan: no {nm}")
        _need(t, nm, torch.float32, 2, contiguous=False)
        if t.shape != (rows, heads * d) or t.stride(1) != 1:
            raise KernelError(f"delta_scan: {nm} {tuple(t.shape)} for {heads} heads of {d}")
    rank, w2_code = 0, F32
    if low is not None:
        _need(low, "decay projection", torch.float32, 2, contiguous=False)
        if w2 is None:
            raise KernelError("delta_scan: the decay's first product without its second matrix")
        _need(w2, "decay matrix", dim=2)
        rank = w2.shape[1]
        if max_q_len != 1 or low.shape != (rows, rank) or low.stride(1) != 1 or w2.shape[0] != heads * d or rank > DELTA_FUSED_MAX_RANK:
            raise KernelError(f"delta_scan: low {tuple(low.shape)}, w2 {tuple(w2.shape)} for rows of up to {max_q_len}")
        w2_code = _code(w2.dtype)
    for t, nm in ((decay_bias, "decay bias"), (remove_bias, "removal bias")):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.numel() != heads * d:
                raise KernelError(f"delta_scan: {nm} of {t.numel()} for {heads} heads of {d}")
    for t, nm in ((seq_slot, "seq_slot"), (seq_q_start, "seq_q_start"), (seq_q_len, "seq_q_len")):
        _need(t, nm, torch.int32, 1)
        if t.numel() < nseq:
            raise KernelError(f"delta_scan: {nm} has {t.numel()} entries for {nseq} sequences")
    single = int(max_q_len) == 1 and not (prepare and low is None)
    dots = None if single else torch.empty((rows, heads, 4), dtype=torch.float32, device=rkv.device)
    p = _DeltaStateParams(rkv.data_ptr(), rkv.stride(0), r_off, k_off, v_off, 0 if decay is None else decay.data_ptr(),
                          0 if decay is None else decay.stride(0), 0 if decay_bias is None else decay_bias.data_ptr(), decay_scale,
                          remove.data_ptr(), remove.stride(0), 0 if remove_bias is None else remove_bias.data_ptr(),
                          0 if low is None else low.data_ptr(), 0 if low is None else low.stride(0), 0 if w2 is None else w2.data_ptr(), rank,
                          key_eps, 0 if dots is None else dots.data_ptr(), state.data_ptr(), state.stride(0), state.stride(1),
                          out.data_ptr(), out.stride(0), seq_slot.data_ptr(), seq_q_start.data_ptr(), seq_q_len.data_ptr(), rows, nseq,
                          heads, d, dv, state.shape[0], int(max_q_len))
    _check(_lib.gb_delta_scan(byref(p), _code(rkv.dtype), c_int(w2_code), _stream()), 1 if single else 2)


def tanh_(z: torch.Tensor) -> None:
    """In place: z = tanh(z), float32 [rows, cols] (the row stride is free)."""
    _need(z, "tanh rows", torch.float32, 2, contiguous=False)
    if z.stride(1) != 1:
        raise KernelError("tanh: rows are not contiguous")
    _check(_lib.gb_tanh(_ptr(z), c_int(z.shape[0]), c_int(z.shape[1]), c_int64(z.stride(0)), _stream()))


# ---- attention with sigmoid weights and a short convolution ahead of it -----------------------
class _ConvQkvParams(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("row_stride", c_int64), ("conv_w", c_void_p), ("taps", c_int), ("channels", c_int),
        ("state", c_void_p), ("state_slot_stride", c_int64), ("qk_norm", c_int), ("v_norm", c_int), ("eps", c_float),
        ("q_out", c_void_p), ("q_out_stride", c_int64), ("row_pos", c_void_p), ("row_seq", c_void_p), ("seq_slot", c_void_p),
        ("seq_q_start", c_void_p), ("seq_q_len", c_void_p), ("block_table", c_void_p), ("bt_stride", c_int),
        ("k_plane", c_void_p), ("v_plane", c_void_p), ("rows", c_int), ("nseq", c_int), ("heads", c_int), ("kv_heads", c_int),
        ("d", c_int), ("dv", c_int), ("pages", c_int), ("max_slots", c_int), ("max_q_len", c_int),
    ]


def conv_qkv(qkv: torch.Tensor, q_out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, value_dim: int,
             conv_weight: Optional[torch.Tensor], state: Optional[torch.Tensor], qk_norm: bool, v_norm: bool, eps: float,
             batch, block_table: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor) -> None:
    """Per row of the projected q | k | v (``qkv``, whose rows may be wider): a causal convolution over time on
    every channel (``conv_weight`` float32 [channels, taps]; None: none), reaching back into the step's earlier
    rows of the same sequence and, before them, into ``state`` (float32 [slots, (taps - 1) * channels], the
    sequence's last projected rows, left updated); each head over its root mean square (``qk_norm``,
    ``v_norm``); q into ``q_out`` [rows, heads * head_dim], k and v into the cache at the row's position."""
    _need(qkv, "qkv", dim=2, contiguous=False)
    _need(q_out, "q out", qkv.dtype, 2, contiguous=False)
    rows = qkv.shape[0]
    channels = (heads + kv_heads) * head_dim + kv_heads * value_dim
    if qkv.stride(1) != 1 or qkv.shape[1] < channels or q_out.shape != (rows, heads * head_dim) or q_out.stride(1) != 1:
        raise KernelError(f"conv_qkv: qkv {tuple(qkv.shape)}, q out {tuple(q_out.shape)} for {heads}+{kv_heads} heads of {head_dim} / {value_dim}")
    taps = 0
    if conv_weight is not None:
        _need(conv_weight, "convolution weights", torch.float32, 2)
        taps = conv_weight.shape[1]
        if conv_weight.shape[0] != channels:
            raise KernelError(f"conv_qkv: convolution weights {tuple(conv_weight.shape)} for {channels} channels")
    slot_stride = 0
    if taps > 1:
        if state is None:
            raise KernelError("conv_qkv: a convolution needs the sequences' state")
        _need(state, "convolution state", torch.float32, 2, contiguous=False)
        if state.shape[1] < (taps - 1) * channels or state.stride(1) != 1:
            raise KernelError(f"conv_qkv: state {tuple(state.shape)} for {taps - 1} rows of {channels}")
        slot_stride = state.stride(0)
    for t, nm, n in ((k_plane, "key plane", head_dim), (v_plane, "value plane", value_dim)):
        _need(t, nm, qkv.dtype, 4)
        if t.shape[1] != kv_heads or t.shape[2] != PAGE or t.shape[3] != n:
            raise KernelError(f"conv_qkv: {nm} {tuple(t.shape)} for {kv_heads} kv heads of {n}")
    _need(block_table, "block table", torch.int32, 2)
    p = _ConvQkvParams(qkv.data_ptr(), qkv.stride(0), 0 if conv_weight is None else conv_weight.data_ptr(), taps, channels,
                       0 if state is None or taps <= 1 else state.data_ptr(), slot_stride, 1 if qk_norm else 0, 1 if v_norm else 0, eps,
                       q_out.data_ptr(), q_out.stride(0), batch.row_pos.data_ptr(), batch.row_seq.data_ptr(),
                       batch.seq_slot.data_ptr(), batch.seq_q_start.data_ptr(), batch.seq_q_len.data_ptr(),
                       block_table.data_ptr(), block_table.stride(0), k_plane.data_ptr(), v_plane.data_ptr(), rows, batch.nseq,
                       heads, kv_heads, head_dim, value_dim, k_plane.shape[0], block_table.shape[0], int(getattr(batch, "max_q_len", 0)))
    _check(_lib.gb_conv_qkv(byref(p), _code(qkv.dtype), _stream()), 2 if taps > 1 and getattr(batch, "max_q_len", 0) != 1 else 1)


class _SigmoidAttnParams(Structure):
    _fields_ = _AttnParams._fields_ + [("score_bias", c_void_p), ("gate", c_void_p), ("gate_stride", c_int64)]


def attention_sigmoid(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor, block_table: torch.Tensor,
                      batch, heads: int, kv_heads: int, head_dim: int, scale: float, window: int = 0,
                      value_dim: Optional[int] = None, score_bias: Optional[torch.Tensor] = None,
                      gate: Optional[torch.Tensor] = None, algo: str = "auto") -> None:
    """Causal grouped-query attention over the paged cache with weights sigmoid((q . k) * scale + score_bias[h])
    that are not normalised over the keys; ``window`` > 0: row i sees keys j with 0 <= i - j < window.  With
    ``gate`` ([rows, heads] pre-activations, a view with a free row stride) head h's output is multiplied by
    sigmoid(gate[row, h]).  out is [rows, heads * value_dim].  bfloat16 rows with key heads of 32, 64, 96 or
    128 and value heads of 32, 48, 64 or 128 run on the tensor cores (prompts of 65 rows and more with heads of
    128 on the tcgen05 kernel, the rest on mma.sync; ``algo`` "mma" asks for mma.sync), everything else (and
    ``algo`` "simt") on the CUDA cores."""
    if algo not in ("auto", "simt", "mma"):
        raise KernelError(f"attention_sigmoid: unknown algorithm '{algo}'")
    a = _attn_params(q, out, k_plane, v_plane, block_table, batch.seq_slot, batch.seq_q_start, batch.seq_q_len, batch.seq_kv_len,
                     batch.nseq, batch.max_q_len, heads, kv_heads, head_dim, scale, window, 1, None, value_dim)
    if score_bias is not None:
        _need(score_bias, "score bias", torch.float32, 1)
        if score_bias.numel() != heads:
            raise KernelError(f"attention_sigmoid: score bias of {score_bias.numel()} for {heads} heads")
    gstride = 0
    if gate is not None:
        _need(gate, "head gates", q.dtype, 2, contiguous=False)
        if gate.shape != (q.shape[0], heads) or gate.stride(1) != 1:
            raise KernelError(f"attention_sigmoid: gates {tuple(gate.shape)} for {q.shape[0]} rows of {heads} heads")
        gstride = gate.stride(0)
    p = _SigmoidAttnParams()
    for name, _ in _AttnParams._fields_:
        setattr(p, name, getattr(a, name))
    p.score_bias = 0 if score_bias is None else score_bias.data_ptr()
    p.gate = 0 if gate is None else gate.data_ptr()
    p.gate_stride = gstride
    if algo == "simt":
        p.num_splits = -1
    elif algo == "mma":
        p.num_splits = -2
    _check(_lib.gb_attention_sigmoid(byref(p), _code(q.dtype), c_int(q.shape[0]), _stream()))


# ---- mixture of experts -----------------------------------------------------------------------
class _MoeRouteParams(Structure):
    _fields_ = [("logits", c_void_p), ("logits_stride", c_int64), ("rows", c_int), ("experts", c_int), ("top", c_int),
                ("renorm_eps", c_float), ("dense", c_void_p), ("index", c_void_p), ("weight", c_void_p), ("score_kind", c_int), ("renorm", c_int)]


class _MoeRowsParams(Structure):
    _fields_ = [("x", c_void_p), ("x_stride", c_int64), ("up", c_void_p), ("down", c_void_p), ("act", c_void_p), ("out", c_void_p),
                ("out_stride", c_int64), ("index", c_void_p), ("weight", c_void_p), ("rows", c_int), ("experts", c_int), ("top", c_int),
                ("ff", c_int), ("hidden", c_int), ("act_kind", c_int), ("weight_input", c_int), ("limit", c_float), ("slope", c_float)]


MOE_SCORES = {"softmax": 0, "sigmoid": 1}
MOE_ACTS = {"relu2": 0, "swiglu": 1, "glu_clamp": 2}     # the last two are gated: an expert's gate rows, then its up rows


def moe_route(logits: torch.Tensor, top: int, renorm_eps: float, dense: torch.Tensor, index: torch.Tensor, weight: torch.Tensor,
              score: str = "softmax", renorm: bool = True) -> None:
    """Per row of ``logits`` (float32 [rows, experts]): scores (softmax over the experts, or with ``score``
    "sigmoid" the sigmoid of each logit by itself), the ``top`` largest chosen, their weights s / (sum of the
    chosen + renorm_eps), or with ``renorm`` False the scores themselves, left in ``dense`` (float32 [rows,
    experts], zeros elsewhere) and as pairs in ``index`` (int32 [rows, top]) and ``weight`` (float32 [rows, top])."""
    _need(logits, "router logits", torch.float32, 2, contiguous=False)
    rows, experts = logits.shape
    _need(dense, "expert weights", torch.float32, 2)
    _need(index, "chosen experts", torch.int32, 2)
    _need(weight, "chosen weights", torch.float32, 2)
    if logits.stride(1) != 1 or dense.shape != (rows, experts) or index.shape != (rows, top) or weight.shape != (rows, top):
        raise KernelError(f"moe_route: logits {tuple(logits.shape)}, dense {tuple(dense.shape)}, pairs {tuple(index.shape)} / {tuple(weight.shape)}")
    p = _MoeRouteParams(logits.data_ptr(), logits.stride(0), rows, experts, top, renorm_eps, dense.data_ptr(), index.data_ptr(), weight.data_ptr(),
                        MOE_SCORES[score], 1 if renorm else 0)
    _check(_lib.gb_moe_route(byref(p), _stream()))


def moe_act(up: torch.Tensor, dense: Optional[torch.Tensor], act: torch.Tensor, experts: int, ff: int, kind: str = "relu2",
            weight_input: bool = False, limit: float = 0.0, slope: float = 1.0) -> None:
    """act[r, e * ff + i] = dense[r, e] * relu(up[r, e * ff + i])^2 (``act`` may be ``up``).  ``kind`` "swiglu": ``up``
    holds, for each expert, ff gate columns and then ff up columns, and the activation is silu(gate) * up (``act`` is
    then another tensor).  ``weight_input``: the weight multiplies the expert's input (its products) instead of its
    result.  ``kind`` "glu_clamp": the same layout, g * sigmoid(slope * g) * (v + 1) with g = min(gate, limit) and
    v = clamp(up, -limit, limit).  ``dense`` None: weights of 1."""
    _need(up, "expert pre-activations", dim=2, contiguous=False)
    _need(act, "expert activations", up.dtype, 2, contiguous=False)
    if dense is not None:
        _need(dense, "expert weights", torch.float32, 2)
    rows = up.shape[0]
    per = 1 if kind == "relu2" else 2
    if (up.shape != (rows, experts * ff * per) or act.shape != (rows, experts * ff) or (dense is not None and dense.shape != (rows, experts))
            or up.stride(1) != 1 or act.stride(1) != 1 or (per == 2 and act.data_ptr() == up.data_ptr())):
        raise KernelError(f"moe_act: up {tuple(up.shape)}, act {tuple(act.shape)} for {experts} experts of {ff} ({kind})")
    _check(_lib.gb_moe_act_clamped(_ptr(up), c_int64(up.stride(0)), _ptr(dense), _ptr(act), c_int64(act.stride(0)), c_int(rows), c_int(experts),
                                   c_int(ff), c_int(MOE_ACTS[kind]), c_int(1 if weight_input else 0), c_float(limit), c_float(slope),
                                   _code(up.dtype), _stream()))


def moe_rows(x: torch.Tensor, up: torch.Tensor, down: torch.Tensor, index: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
             experts: int, ff: int, kind: str = "relu2", weight_input: bool = False, limit: float = 0.0, slope: float = 1.0) -> None:
    """The experts' feed-forward for a step of few rows, reading only the chosen experts' matrices:
    out[r] = sum_k weight[r, k] * down_e(relu(up_e x[r])^2), e = index[r, k].  ``up`` is [experts * ff, hidden]
    (the up matrices one above the other), ``down`` [hidden, experts * ff] (the down matrices side by side),
    ``out`` float32 [rows, hidden].  ``kind`` "swiglu": gated experts, ``up`` [experts * 2 ff, hidden] with each
    expert's gate rows ahead of its up rows; ``weight_input``: the weight multiplies the expert's input."""
    per = 1 if kind == "relu2" else 2
    _need(x, "moe x", dim=2, contiguous=False)
    _need(up, "stacked up matrices", dim=2)
    _need(down, "stacked down matrices", up.dtype, 2)
    _need(out, "moe out", torch.float32, 2, contiguous=False)
    _need(index, "chosen experts", torch.int32, 2)
    _need(weight, "chosen weights", torch.float32, 2)
    rows, hidden = x.shape
    top = index.shape[1]
    if (up.shape != (experts * ff * per, hidden) or down.shape != (hidden, experts * ff) or out.shape != (rows, hidden) or x.stride(1) != 1
            or out.stride(1) != 1 or index.shape[0] != rows or weight.shape != index.shape):
        raise KernelError(f"moe_rows: x {tuple(x.shape)}, up {tuple(up.shape)}, down {tuple(down.shape)}, out {tuple(out.shape)}")
    act = torch.empty((rows, top, ff), dtype=x.dtype, device=x.device)
    p = _MoeRowsParams(x.data_ptr(), x.stride(0), up.data_ptr(), down.data_ptr(), act.data_ptr(), out.data_ptr(), out.stride(0),
                       index.data_ptr(), weight.data_ptr(), rows, experts, top, ff, hidden, MOE_ACTS[kind], 1 if weight_input else 0, limit, slope)
    _check(_lib.gb_moe_rows(byref(p), _code(x.dtype), _code(up.dtype), _stream()), 2)


def moe_rows_grouped(x: torch.Tensor, up: torch.Tensor, down: torch.Tensor, offsets: torch.Tensor, src_row: torch.Tensor, ys: torch.Tensor,
                     experts: int, top: int, ff: int, kind: str = "relu2", sorted_weight: Optional[torch.Tensor] = None,
                     limit: float = 0.0, slope: float = 1.0) -> None:
    """The few-row feed-forward with the (row, choice) pairs sorted by expert (``offsets`` and ``src_row`` from
    ``moe_group``): every expert's matrices are read once, ``ys`` (float32 [rows * top, hidden]) receives each pair's
    output down_e(relu(up_e x)^2) at its sorted place; ``moe_combine`` adds a row's pairs up with their weights.
    ``kind`` as for ``moe_rows``; ``sorted_weight`` (float32 [rows * top], the pairs' weights in sorted order): the
    weight multiplies the expert's input here, and ``moe_combine`` then adds up without weights."""
    per = 1 if kind == "relu2" else 2
    if sorted_weight is not None:
        _need(sorted_weight, "sorted weights", torch.float32, 1)
    _need(x, "moe x", dim=2, contiguous=False)
    _need(up, "stacked up matrices", dim=2)
    _need(down, "stacked down matrices", up.dtype, 2)
    _need(ys, "expert outputs", torch.float32, 2)
    _need(offsets, "offsets", torch.int32, 1)
    _need(src_row, "source rows", torch.int32, 1)
    rows, hidden = x.shape
    if (up.shape != (experts * ff * per, hidden) or down.shape != (hidden, experts * ff) or ys.shape != (rows * top, hidden) or x.stride(1) != 1
            or offsets.numel() < experts + 1 or src_row.numel() < rows * top or (sorted_weight is not None and sorted_weight.numel() < rows * top)):
        raise KernelError(f"moe_rows_grouped: x {tuple(x.shape)}, up {tuple(up.shape)}, down {tuple(down.shape)}, outputs {tuple(ys.shape)}")
    act = torch.empty((rows * top, ff), dtype=x.dtype, device=x.device)
    p = _MoeRowsParams(x.data_ptr(), x.stride(0), up.data_ptr(), down.data_ptr(), act.data_ptr(), 0, 0, 0,
                       0 if sorted_weight is None else sorted_weight.data_ptr(), rows, experts, top, ff, hidden, MOE_ACTS[kind],
                       0 if sorted_weight is None else 1, limit, slope)
    _check(_lib.gb_moe_rows_grouped(byref(p), _ptr(offsets), _ptr(src_row), _ptr(ys), _code(x.dtype), _code(up.dtype), _stream()), 2)


def moe_group(index: torch.Tensor, experts: int, offsets: torch.Tensor, place: torch.Tensor, src_row: torch.Tensor,
              weight: Optional[torch.Tensor] = None, sorted_weight: Optional[torch.Tensor] = None) -> None:
    """Sort the (row, choice) pairs of ``index`` (int32 [rows, top]) by expert: ``offsets`` (int32 [experts + 1]) receives
    where each expert's group starts, ``place`` (int32 [rows * top]) each pair's position in the sorted order and
    ``src_row`` (int32 [rows * top]) the row of the pair at each position.  With ``weight`` (float32 [rows, top]) and
    ``sorted_weight`` (float32 [rows * top]) the pairs' weights are left in sorted order too."""
    _need(index, "chosen experts", torch.int32, 2)
    rows, top = index.shape
    for t, nm, n in ((offsets, "offsets", experts + 1), (place, "places", rows * top), (src_row, "source rows", rows * top)):
        _need(t, nm, torch.int32, 1)
        if t.numel() < n:
            raise KernelError(f"moe_group: {nm} has {t.numel()} entries, want {n}")
    if (weight is None) != (sorted_weight is None):
        raise KernelError("moe_group: weights in and out go together")
    if weight is not None:
        _need(weight, "chosen weights", torch.float32, 2)
        _need(sorted_weight, "sorted weights", torch.float32, 1)
        if weight.shape != index.shape or sorted_weight.numel() < rows * top:
            raise KernelError(f"moe_group: weights {tuple(weight.shape)} / {sorted_weight.numel()} for pairs {tuple(index.shape)}")
    _check(_lib.gb_moe_group_weights(_ptr(index), c_int(rows), c_int(top), c_int(experts), _ptr(offsets), _ptr(place), _ptr(src_row),
                                     _ptr(weight), _ptr(sorted_weight), _stream()))


def moe_gather(x: torch.Tensor, src_row: torch.Tensor, xs: torch.Tensor) -> None:
    """xs[p] = x[src_row[p]]."""
    _need(x, "moe x", dim=2, contiguous=False)
    _need(xs, "gathered rows", x.dtype, 2)
    _need(src_row, "source rows", torch.int32, 1)
    if xs.shape[1] != x.shape[1] or src_row.numel() < xs.shape[0] or x.stride(1) != 1:
        raise KernelError(f"moe_gather: x {tuple(x.shape)}, gathered {tuple(xs.shape)}, {src_row.numel()} source rows")
    _check(_lib.gb_moe_gather(_ptr(x), c_int64(x.stride(0)), _ptr(src_row), _ptr(xs), c_int(xs.shape[0]), c_int(x.shape[1]), _code(x.dtype), _stream()))


def relu2(z: torch.Tensor) -> None:
    """In place: z = max(z, 0)^2."""
    _need(z, "relu2 rows")
    _check(_lib.gb_relu2(_ptr(z), c_int64(z.numel()), _code(z.dtype), _stream()))


def moe_combine(ys: torch.Tensor, place: torch.Tensor, weight: Optional[torch.Tensor], out: torch.Tensor, top: Optional[int] = None) -> None:
    """out[r] = sum_k weight[r, k] * ys[place[r * top + k]], float32, in the order of k (``weight`` None: the plain
    sum of ``top`` outputs a row)."""
    _need(ys, "expert outputs", torch.float32, 2)
    _need(place, "places", torch.int32, 1)
    _need(out, "moe out", torch.float32, 2, contiguous=False)
    if weight is not None:
        _need(weight, "chosen weights", torch.float32, 2)
        rows, top = weight.shape
    else:
        rows, top = out.shape[0], int(top)
    if out.shape != (rows, ys.shape[1]) or ys.shape[0] != rows * top or place.numel() < rows * top or out.stride(1) != 1:
        raise KernelError(f"moe_combine: outputs {tuple(ys.shape)}, {rows} x {top} pairs, out {tuple(out.shape)}")
    _check(_lib.gb_moe_combine(_ptr(ys), _ptr(place), _ptr(weight), _ptr(out), c_int64(out.stride(0)), c_int(rows), c_int(top), c_int(ys.shape[1]),
                               _stream()))


def gemm_w_cols(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> str:
    """out = a @ w^T where ``w`` may be a block of columns of a wider matrix (its rows lie ``w.stride(0)`` apart): the
    tiled tcgen05 kernels for aligned bfloat16 operands, else the CUDA-core kernel.  Returns the kernel's name."""
    _need(a, "gemm a", dim=2, contiguous=False)
    _need(w, "gemm w", dim=2, contiguous=False)
    _need(out, "gemm out", dim=2, contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    fits = (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.dtype in (torch.float32, torch.bfloat16))
    if not fits:
        _check(_lib.gb_gemm_simt(_ptr(a), _code(a.dtype), _ptr(w), _code(w.dtype), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                 c_int64(a.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0)), _stream()))
        return "simt"
    pair = M >= TC5_PAIR_MIN_ROWS
    _check(_lib.gb_gemm_tc5_ldw(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K), c_int64(a.stride(0)),
                                c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(1 if pair else 0), _stream()))
    return "tc5_pair" if pair else "tc5"


def gemm_grouped_fits(a_dtype, w: torch.Tensor, K: int, by_cols: bool) -> bool:
    """Whether ``gemm_grouped`` takes these operands: bfloat16, rows and blocks that start on 16 bytes."""
    return (a_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0
            and w.data_ptr() % 16 == 0)


def gemm_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor, groups: int, *, by_cols: bool = False,
                 gated: bool = False, row_weight: Optional[torch.Tensor] = None, row_map: Optional[torch.Tensor] = None,
                 gate: str = "swiglu", limit: float = 0.0, slope: float = 1.0) -> None:
    """One launch for the products of every group of rows: rows ``offsets[e] .. offsets[e + 1] - 1`` of ``a`` [P, K]
    (sorted by group; ``offsets`` int32 [groups + 1] on the device, never read on the host) times block e of ``w``.
    ``by_cols`` False: ``w`` is [groups * block, K] and block e its rows e * block ..; with ``gated`` a block is N gate
    rows, then N up rows, and out = silu(f g) * (f u), f = ``row_weight[row]`` (1 if absent), or with ``gate`` "glu_clamp"
    c * sigmoid(slope * c) * (v + 1), c = min(f g, limit), v = clamp(f u, -limit, limit).  ``by_cols`` True: ``w`` is
    [N, groups * K] and block e its columns e * K ...  ``out`` is [*, N]; with ``row_map`` (int32 [P]) the result of
    row r is written to row ``row_map[r]`` of ``out``, otherwise to row r."""
    _need(a, "grouped gemm a", torch.bfloat16, 2, contiguous=False)
    _need(w, "grouped gemm w", torch.bfloat16, 2, contiguous=False)
    _need(out, "grouped gemm out", dim=2, contiguous=False)
    _need(offsets, "group offsets", torch.int32, 1)
    P, K = a.shape
    N = out.shape[1]
    if offsets.numel() < groups + 1 or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm_grouped: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, {offsets.numel()} offsets")
    if by_cols:
        if gated or w.shape != (N, groups * K):
            raise KernelError(f"gemm_grouped: w {tuple(w.shape)} is not [{N}, {groups} x {K}]")
        block = 0
    else:
        if w.shape[0] % groups or w.shape[1] != K or w.shape[0] // groups != (2 * N if gated else N):
            raise KernelError(f"gemm_grouped: w {tuple(w.shape)} is not {groups} blocks of {2 * N if gated else N} rows of {K}")
        block = w.shape[0] // groups
    if row_map is None and out.shape[0] < P:
        raise KernelError(f"gemm_grouped: out has {out.shape[0]} rows for {P}")
    if row_weight is not None:
        _need(row_weight, "row weights", torch.float32, 1)
        if row_weight.numel() < P or not gated:
            raise KernelError("gemm_grouped: row weights go with gated outputs, one a row")
    if row_map is not None:
        _need(row_map, "row map", torch.int32, 1)
        if row_map.numel() < P:
            raise KernelError(f"gemm_grouped: {row_map.numel()} mapped rows for {P}")
    if gate not in ("swiglu", "glu_clamp"):
        raise KernelError(f"gemm_grouped: unknown gate '{gate}'")
    _check(_lib.gb_gemm_tc5_grouped_act(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), _ptr(offsets), c_int(groups), c_int(P), c_int(N), c_int(K),
                                        c_int64(a.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(block), c_int(1 if by_cols else 0),
                                        c_int(0 if not gated else (2 if gate == "glu_clamp" else 1)), _ptr(row_weight), _ptr(row_map),
                                        c_float(limit), c_float(slope), _stream()))


# ---- layers with the norm behind the sublayer, differential and latent attention ----------------
def norm_scale_add(h: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, x_out: Optional[torch.Tensor] = None) -> None:
    """h += y / sqrt(mean(y^2) + eps) * weight on float32 rows (``weight``: the norm's weight with the sublayer's
    constant factors folded in); with ``x_out`` the new rows are left there too, in its dtype, for whoever reads
    the residual next."""
    _need(h, "residual", torch.float32, 2)
    _need(y, "sublayer output", torch.float32, 2)
    _need(weight, "norm weight", torch.float32, 1)
    rows, n = h.shape
    if y.shape != h.shape or weight.numel() != n:
        raise KernelError(f"norm_scale_add: h {tuple(h.shape)}, y {tuple(y.shape)}, weight {tuple(weight.shape)}")
    if x_out is not None:
        _need(x_out, "rows out", dim=2)
        if x_out.shape != h.shape:
            raise KernelError(f"norm_scale_add: rows out {tuple(x_out.shape)} for h {tuple(h.shape)}")
    _check(_lib.gb_norm_scale_add(_ptr(h), _ptr(y), _ptr(weight), c_float(eps), c_int(rows), c_int(n), _ptr(x_out),
                                  c_int(F32 if x_out is None else _code(x_out.dtype)), _stream()))


def diff_combine(ctx: torch.Tensor, out: torch.Tensor, heads: int, per_group: int, value_dim: int, lam: float, eps: float, factor: float) -> None:
    """The two softmax maps of every head combined: o = a1 - lam * a2, o / sqrt(mean(o^2) + eps) * factor.  ``ctx`` is
    the attention output [rows, 2 * heads * value_dim] with the heads of a key group ordered [map 1 of each of its
    ``per_group`` heads, map 2 of each]; ``out`` [rows, heads * value_dim] in the model's head order."""
    _need(ctx, "attention maps", dim=2, contiguous=False)
    _need(out, "combined heads", ctx.dtype, 2, contiguous=False)
    rows = ctx.shape[0]
    if (ctx.shape[1] != 2 * heads * value_dim or out.shape != (rows, heads * value_dim) or ctx.stride(1) != 1 or out.stride(1) != 1
            or per_group <= 0 or heads % per_group):
        raise KernelError(f"diff_combine: maps {tuple(ctx.shape)}, out {tuple(out.shape)} for {heads} heads of {value_dim} in groups of {per_group}")
    _check(_lib.gb_diff_combine(_ptr(ctx), c_int64(ctx.stride(0)), _ptr(out), c_int64(out.stride(0)), c_int(rows), c_int(heads), c_int(per_group),
                                c_int(value_dim), c_float(lam), c_float(eps), c_float(factor), _code(ctx.dtype), _stream()))


def add_rows_gated(out: torch.Tensor, y: torch.Tensor, z: torch.Tensor) -> None:
    """out[r] += sigmoid(z[r]) * y[r]; ``z`` float32 [rows] (a view with a free stride)."""
    _need(out, "sum", torch.float32, 2)
    _need(y, "addend", torch.float32, 2)
    _need(z, "gate", torch.float32, 1, contiguous=False)
    if y.shape != out.shape or z.numel() != out.shape[0]:
        raise KernelError(f"add_rows_gated: out {tuple(out.shape)}, y {tuple(y.shape)}, gate {tuple(z.shape)}")
    _check(_lib.gb_add_rows_gated(_ptr(out), _ptr(y), _ptr(z), c_int64(z.stride(0)), c_int(out.shape[0]), c_int(out.shape[1]), _stream()))


def latent_prep(lat: torch.Tensor, cq: torch.Tensor, q_weight: torch.Tensor, kv_weight: torch.Tensor, eps: float, cos: Optional[torch.Tensor],
                sin: Optional[torch.Tensor], q_rank: int, kv_rank: int, rot: int, row_pos: torch.Tensor, row_seq: torch.Tensor,
                seq_slot: torch.Tensor, block_table: torch.Tensor, k_plane: Optional[torch.Tensor], write_kv: bool) -> None:
    """Rows of a fused down-projection [q latent | kv latent | rotated key part]: the q latent RMS-normed with
    ``q_weight`` into ``cq``; the kv latent RMS-normed with ``kv_weight`` and the key part rotated (channels 2j and
    2j + 1 by angle j of the tables) into ``k_plane`` ([pages, 1, 64, kv_rank + rot]) at each row's position."""
    _need(lat, "latents", dim=2, contiguous=False)
    _need(cq, "q latent", lat.dtype, 2)
    _need(q_weight, "q latent norm", torch.float32, 1)
    _need(kv_weight, "kv latent norm", torch.float32, 1)
    rows = lat.shape[0]
    if (lat.shape[1] < q_rank + kv_rank + rot or lat.stride(1) != 1 or cq.shape != (rows, q_rank) or q_weight.numel() != q_rank
            or kv_weight.numel() != kv_rank):
        raise KernelError(f"latent_prep: latents {tuple(lat.shape)}, q latent {tuple(cq.shape)} for ranks {q_rank}, {kv_rank} and {rot} rotated channels")
    tp = 0
    if rot > 0:
        _need(cos, "rope cos", torch.float32, 2)
        _need(sin, "rope sin", torch.float32, 2)
        if cos.shape[1] != rot // 2 or sin.shape != cos.shape:
            raise KernelError(f"latent_prep: angle tables {tuple(cos.shape)} for {rot} rotated channels")
        tp = cos.shape[0]
    for t, nm in ((row_pos, "row_pos"), (row_seq, "row_seq"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if write_kv:
        _need(k_plane, "key plane", lat.dtype, 4)
        if tuple(k_plane.shape[1:]) != (1, PAGE, kv_rank + rot):
            raise KernelError(f"latent_prep: key plane {tuple(k_plane.shape)} for a latent of {kv_rank} + {rot}")
    _check(_lib.gb_latent_prep(_ptr(lat), c_int64(lat.stride(0)), _ptr(cq), _ptr(q_weight), _ptr(kv_weight), c_float(eps), _ptr(cos), _ptr(sin),
                               c_int(tp), _ptr(row_pos), _ptr(row_seq), _ptr(seq_slot), _ptr(block_table), c_int(block_table.stride(0)),
                               _ptr(k_plane if write_kv else None), c_int(1 if write_kv else 0), c_int(rows), c_int(q_rank), c_int(kv_rank),
                               c_int(rot), c_int(k_plane.shape[0] if write_kv else 0), c_int(block_table.shape[0]), _code(lat.dtype), _stream()))


def latent_q_rot(q: torch.Tensor, out: torch.Tensor, heads: int, head_dim: int, rot: int, cos: torch.Tensor, sin: torch.Tensor,
                 row_pos: torch.Tensor) -> None:
    """The last ``rot`` channels of every query head of ``q`` ([rows, heads * (head_dim + rot)]) rotated by the row's
    position (channels 2j and 2j + 1 together) into the last ``rot`` channels of every head of ``out``
    ([rows, heads * out_head])."""
    _need(q, "queries", dim=2, contiguous=False)
    _need(out, "absorbed queries", q.dtype, 2, contiguous=False)
    rows = q.shape[0]
    if rot <= 0:
        return
    out_head = out.shape[1] // heads
    if q.shape[1] != heads * (head_dim + rot) or out.shape[1] != heads * out_head or out_head < rot or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"latent_q_rot: q {tuple(q.shape)}, out {tuple(out.shape)} for {heads} heads of {head_dim} + {rot}")
    _need(cos, "rope cos", torch.float32, 2)
    _need(sin, "rope sin", torch.float32, 2)
    _need(row_pos, "row_pos", torch.int32, 1)
    if cos.shape[1] != rot // 2 or sin.shape != cos.shape:
        raise KernelError(f"latent_q_rot: angle tables {tuple(cos.shape)} for {rot} rotated channels")
    _check(_lib.gb_latent_q_rot(_ptr(q), c_int64(q.stride(0)), _ptr(out), c_int64(out.stride(0)), c_int(rows), c_int(heads), c_int(head_dim),
                                c_int(rot), c_int(out_head), _ptr(cos), _ptr(sin), c_int(cos.shape[0]), _ptr(row_pos), _code(q.dtype), _stream()))


HEAD_GEMM_MAX_K = 2048     # float32 rows of this many channels are what one CTA of the kernel stages


def head_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, h, :] = a[r, h, :] @ w[h] for every head in one launch: ``a`` [rows, heads, K] and ``out``
    [rows, heads, N] may be views with free row and head strides, ``w`` is [heads, K, N]; float32 sums on the
    CUDA cores."""
    _need(a, "head_gemm a", dim=3, contiguous=False)
    _need(w, "head_gemm w", dim=3)
    _need(out, "head_gemm out", a.dtype, 3, contiguous=False)
    rows, heads, K = a.shape
    N = w.shape[2]
    if w.shape != (heads, K, N) or out.shape != (rows, heads, N) or a.stride(2) != 1 or out.stride(2) != 1 or K > HEAD_GEMM_MAX_K:
        raise KernelError(f"head_gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check(_lib.gb_head_gemm(_ptr(a), c_int64(a.stride(0)), c_int64(a.stride(1)), _ptr(w), _ptr(out), c_int64(out.stride(0)), c_int64(out.stride(1)),
                             c_int(rows), c_int(heads), c_int(K), c_int(N), _code(a.dtype), _code(w.dtype), _stream()))


def head_gemm_mma_accepts(a: torch.Tensor, w_nk: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether ``head_gemm_mma`` takes these operands (bfloat16, 16-byte aligned rows, even output strides)."""
    if not (a.dtype == w_nk.dtype == out.dtype == torch.bfloat16) or a.dim() != 3 or a.stride(2) != 1 or out.stride(2) != 1:
        return False
    return bool(_lib.gb_head_gemm_mma_accepts(_ptr(a), c_int64(a.stride(0)), c_int64(a.stride(1)), _ptr(w_nk), _ptr(out), c_int64(out.stride(0)),
                                              c_int64(out.stride(1)), c_int(a.shape[2]), c_int(w_nk.shape[1])))


def head_gemm_mma(a: torch.Tensor, w_nk: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, h, :] = a[r, h, :] @ w_nk[h]^T for every head in one launch on the tensor cores: ``a`` [rows, heads, K] and
    ``out`` [rows, heads, N] may be views with free row and head strides, ``w_nk`` is [heads, N, K]; bfloat16."""
    _need(a, "head_gemm a", torch.bfloat16, 3, contiguous=False)
    _need(w_nk, "head_gemm w", torch.bfloat16, 3)
    _need(out, "head_gemm out", torch.bfloat16, 3, contiguous=False)
    rows, heads, K = a.shape
    N = w_nk.shape[1]
    if w_nk.shape != (heads, N, K) or out.shape != (rows, heads, N) or a.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError(f"head_gemm_mma: a {tuple(a.shape)}, w {tuple(w_nk.shape)}, out {tuple(out.shape)}")
    _check(_lib.gb_head_gemm_mma(_ptr(a), c_int64(a.stride(0)), c_int64(a.stride(1)), _ptr(w_nk), _ptr(out), c_int64(out.stride(0)),
                                 c_int64(out.stride(1)), c_int(rows), c_int(heads), c_int(K), c_int(N), _stream()))
