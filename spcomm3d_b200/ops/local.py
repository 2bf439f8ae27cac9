"""Local (single-rank) kernels behind one interface.

Each op takes torch tensors and runs the hand-written sm_100a kernel when the
tensors live on a GPU (csrc/kernels, through libsp3cuda.so) and the OpenMP
C++ loop when they live on the host (csrc/host/cpu_ops.cpp, the path of the
CPU/gloo plumbing configuration).  There is no other implementation behind
these names: if the CUDA library cannot be loaded on a GPU box the call
raises.

Reference loops: sddmm / spmm src/core_ops.cpp:5-35; pack, unpack and
scatter-add of staging buffers src/comm.hpp:90-103,166-189.
"""
from __future__ import annotations

import torch

from ..utils import native

_F = {torch.float32: "f32", torch.float64: "f64"}


def _suffix(t: torch.Tensor) -> str:
    try:
        return _F[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _row_major(t: torch.Tensor):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("dense operand must be 2-D with unit inner stride")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def sddmm(rowidx, colidx, svals, A, B, out=None):
    """out[i] = svals[i] * dot(A[rowidx[i]], B[colidx[i]]); svals may be None."""
    nnz = rowidx.shape[0]
    if out is None:
        out = torch.empty(nnz, dtype=A.dtype, device=A.device)
    if nnz == 0:
        return out
    k = A.shape[1]
    if A.is_cuda:
        from . import cuda_ops
        return cuda_ops.sddmm(rowidx, colidx, svals, A, B, out)
    fn = getattr(native.host(), f"sp3_cpu_sddmm_{_suffix(A)}")
    native.check(fn(nnz, native.ptr(rowidx), native.ptr(colidx), native.ptr(svals), native.ptr(A),
                    _row_major(A), native.ptr(B), _row_major(B), k, native.ptr(out)), "cpu sddmm")
    return out


def spmm(rowptr, rowidx, colidx, vals, X, Y, beta: float = 0.0, sched=None):
    """Y[r] = beta*Y[r] + sum_p vals[p] * X[colidx[p]] over CSR rows r."""
    nrows = rowptr.shape[0] - 1
    if nrows == 0:
        return Y
    k = X.shape[1]
    if X.is_cuda:
        from . import cuda_ops
        return cuda_ops.spmm(rowptr, rowidx, colidx, vals, X, Y, beta, sched)
    fn = getattr(native.host(), f"sp3_cpu_spmm_{_suffix(X)}")
    native.check(fn(nrows, native.ptr(rowptr), native.ptr(colidx), native.ptr(vals), native.ptr(X),
                    _row_major(X), k, float(beta), native.ptr(Y), _row_major(Y)), "cpu spmm")
    return Y


def _rows(mode: int, idx, src, dst):
    n = idx.shape[0]
    if n == 0:
        return dst
    k = src.shape[1]
    if src.is_cuda:
        from . import cuda_ops
        return cuda_ops.rows(mode, idx, src, dst)
    fn = getattr(native.host(), f"sp3_cpu_rows_{_suffix(src)}")
    native.check(fn(mode, n, native.ptr(idx), native.ptr(src), _row_major(src), native.ptr(dst),
                    _row_major(dst), k), "cpu rows")
    return dst


def gather_rows(idx, src, dst):
    """dst[i] = src[idx[i]]  (pack a send buffer)."""
    return _rows(0, idx, src, dst)


def scatter_rows(idx, src, dst):
    """dst[idx[i]] = src[i]  (unpack a receive buffer)."""
    return _rows(1, idx, src, dst)


def scatter_add_rows(idx, src, dst):
    """dst[idx[i]] += src[i]; idx has no repeats (owner-side sum of partial rows)."""
    return _rows(2, idx, src, dst)
