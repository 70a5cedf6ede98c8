"""Matrix products  y = x W^T  (weights row-major [out, in], models/llama/common/src/lib.rs:168-180).

float32: always the CUDA-core kernel of this package (plain FFMA: no reduced-precision matrix mode can slip in).
bfloat16, by the number of rows:
  * up to 16 rows (decoding): ``gemm_skinny``, which streams the weights once through the tensor cores; the experts
    of up to 64 (token, expert) pairs too, with the rows unsorted (``row_group``);
  * more rows, one dense weight: the library (cuBLAS through ``torch.mm``), as the reference hands its ``mat_mul``
    to an operator library (compute.rs:425-455);
  * more rows, grouped (the experts of prompts and of wide decode batches) or float output (logits of many rows):
    ``gemm_tc``, this package's tcgen05 kernel.
"""
from __future__ import annotations

import torch

from ..csrc import lib


def gemm_simt(a, w, out, *, a_rows=None, group_offsets=None, groups=1, rows=None, out_kind=0) -> None:
    """out[m] = a[a_rows[m] or m] . w[g(m)]^T ; w is [N, K] or [G, N(or 2N), K]."""
    M = out.shape[0] if rows is None else rows
    K = a.shape[-1]
    N = out.shape[-1]
    if w.dim() == 3:
        stride = w.stride(0)
        ldb = w.stride(1)
    else:
        stride = 0
        ldb = w.stride(0)
    assert a.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1
    lib.call("tb_gemm_simt_" + lib.suffix(a.dtype), lib.ptr(a), lib.ptr(a_rows), lib.ptr(w), lib.ptr(out),
             lib.ptr(group_offsets), stride, a.stride(0), ldb, out.stride(0), M, N, K, groups, out_kind)


DENSE_TC = False           # dense bfloat16 products of many rows: this package's tcgen05 kernel instead of cuBLAS
SKINNY_MAX_ROWS = 16       # dense: up to this many rows the weight-streaming kernel is used
SKINNY_MAX_PAIRS = 64      # grouped: up to this many rows over all groups (measured in the decode step: the
                           # tensor-core kernel wins from 96 (token, expert) pairs on, by 5 %; below, this one by 5..8 %)


def gemm_skinny(a, w, out, *, a_rows=None, group_offsets=None, groups=1, out_kind=0, max_group_rows=0,
                row_group=None, x_div=1, w_is_weight=True) -> bool:
    """The decode kernel (bfloat16, tensor cores, weights streamed once).  False if it refuses the sizes.
    With ``row_group`` ([M] int32) the rows are unsorted: row m belongs to group row_group[m], reads
    a[m // x_div] and writes out[m] (no offsets, no gathered rows).  ``w_is_weight=False``: ``w`` was computed by
    an earlier kernel of the step (the kernel then reads none of it before that kernel has finished)."""
    M, K, N = out.shape[0], a.shape[-1], out.shape[-1]
    if w.dim() == 3:
        stride, ldw = w.stride(0), w.stride(1)
    else:
        stride, ldw = 0, w.stride(0)
    assert a.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1
    return lib.try_call("tb_gemm_skinny_bf16", lib.ptr(a), lib.ptr(a_rows), lib.ptr(w), lib.ptr(out),
                        lib.ptr(group_offsets), stride, a.stride(0), ldw, out.stride(0), M, N, K, groups, out_kind,
                        max_group_rows, lib.ptr(row_group), x_div, 1 if w_is_weight else 0)


def gemm_tc(a, w, out, *, group_offsets=None, groups=1, out_kind=0) -> bool:
    """The prompt kernel (bfloat16, tcgen05 + TMA + TMEM).  Rows of ``a`` are already sorted by group.
    False if it refuses the sizes."""
    M, K, N = out.shape[0], a.shape[-1], out.shape[-1]
    ldw = w.stride(1) if w.dim() == 3 else w.stride(0)
    assert a.stride(-1) == 1 and w.stride(-1) == 1 and out.stride(-1) == 1 and w.is_contiguous()
    return lib.try_call("tb_gemm_tc_bf16", lib.ptr(a), lib.ptr(w), lib.ptr(out), lib.ptr(group_offsets),
                        a.stride(0), ldw, out.stride(0), M, N, K, groups, out_kind)


def matmul_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, w_is_weight: bool = True) -> None:
    """out = a @ w.T for one dense weight; out has a's type, or float (logits).  ``w`` is taken to be a weight,
    which no kernel of the step writes: the decode kernel starts reading it before the kernel that produced ``a``
    has finished.  Pass ``w_is_weight=False`` if ``w`` is itself a result of the step."""
    M = a.shape[0]
    if M == 0:
        return
    to_float = out.dtype == torch.float32
    if a.dtype == torch.float32:
        gemm_simt(a, w, out, out_kind=0)
        return
    if M <= SKINNY_MAX_ROWS and gemm_skinny(a, w, out, out_kind=1 if to_float else 0, w_is_weight=w_is_weight):
        return
    if (to_float or DENSE_TC) and gemm_tc(a, w, out, out_kind=1 if to_float else 0):
        return
    if to_float:
        gemm_simt(a, w, out, out_kind=1)
    else:
        lib.foreign("mm", a, w, out)       # a recording repeats it with the other layers' own weight
        torch.mm(a, w.t(), out=out)


def grouped_matmul(a, w, out, *, a_rows=None, group_offsets=None, groups=1, swiglu=False, max_group_rows=0,
                   scratch=None, w_is_weight: bool = True) -> None:
    """out[m] = a[a_rows[m] or m] . w[g(m)]^T over rows sorted by group; with swiglu, w[g] holds gate rows
    then up rows and out = silu(gate) * up.  max_group_rows: a bound on the rows of one group, if known;
    scratch(name, shape, dtype): where the prompt kernel may put the gathered rows."""
    kind = 2 if swiglu else 0
    if a.dtype == torch.bfloat16 and out.shape[0] <= SKINNY_MAX_PAIRS and \
            gemm_skinny(a, w, out, a_rows=a_rows, group_offsets=group_offsets, groups=groups, out_kind=kind,
                        max_group_rows=max_group_rows, w_is_weight=w_is_weight):
        return
    if a.dtype == torch.bfloat16 and w.is_contiguous():
        src = a
        if a_rows is not None:
            # TMA fetches tiles of consecutive rows: bring the rows into their sorted order first
            src = None
            if scratch is not None:
                buf = scratch("grouped.sorted_rows", (out.shape[0], a.shape[-1]), a.dtype)
                if lib.try_call("tb_gather_rows_bf16", lib.ptr(a), lib.ptr(a_rows), lib.ptr(buf), out.shape[0],
                                a.shape[-1]):
                    src = buf
        if src is not None and gemm_tc(src, w, out, group_offsets=group_offsets, groups=groups, out_kind=kind):
            return
    gemm_simt(a, w, out, a_rows=a_rows, group_offsets=group_offsets, groups=groups, out_kind=kind)
