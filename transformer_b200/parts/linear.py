"""Matrix products  y = x W^T  (weights row-major [out, in], models/llama/common/src/lib.rs:168-180).

float32: always the CUDA-core kernel of this package (plain FFMA: no reduced-precision matrix mode
can slip in).  bfloat16: dense products go to the library (cuBLAS through ``torch.mm``), as the
reference hands its ``mat_mul`` to an operator library (compute.rs:425-455); grouped products (the
experts) and products with float output use this package's kernels.
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


def matmul_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = a @ w.T for one dense weight; out has a's type, or float (logits)."""
    if a.shape[0] == 0:
        return
    if a.dtype == torch.float32:
        gemm_simt(a, w, out, out_kind=0)
    elif out.dtype == torch.float32:
        gemm_simt(a, w, out, out_kind=1)
    else:
        torch.mm(a, w.t(), out=out)
