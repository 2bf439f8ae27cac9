"""The allocation-free SpMM entry point, called through its exported C symbol.

Some users of the kernel library may not allocate device memory at call time
(a host application that owns the whole memory budget, a callback that must
not touch an allocator, a C program without torch); for them
`sp3_cuda_spmm_f32_noalloc` keeps its scratch in a fixed array inside the
library.  This test checks that it computes what the regular entry point
computes, twice in a row (the second call meets the first call's leftovers in
the shared scratch), and that it refuses a problem that does not fit.

The file sorts last on purpose so that a `-x` run reaches it after all other
tests.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(seed, k, long_rows=(600, 1100, 2100, 513), ld=None):
    rng = np.random.default_rng(seed)
    nrows, ncols = 2000, 1500
    deg = rng.poisson(5, nrows)
    if long_rows:
        deg[rng.choice(nrows, len(long_rows), replace=False)] = long_rows
    rowptr = torch.zeros(nrows + 1, dtype=torch.int64)
    rowptr[1:] = torch.from_numpy(np.cumsum(deg))
    nnz = int(rowptr[-1])
    colidx = torch.from_numpy(rng.integers(0, ncols, nnz).astype(np.int32))
    vals = torch.from_numpy(rng.random(nnz).astype(np.float32))
    ld = k if ld is None else ld   # ld > k: X and Y are column slices of wider buffers
    X = torch.from_numpy(rng.standard_normal((ncols, ld)).astype(np.float32)).cuda()[:, :k]
    Y0 = torch.from_numpy(rng.standard_normal((nrows, ld)).astype(np.float32)).cuda()[:, :k]
    return rowptr.cuda(), colidx.cuda(), vals.cuda(), X, Y0


def _fp64(rowptr, colidx, vals, X, Y0, beta):
    """Y = beta*Y0 + A X with torch in fp64 (the plain reference of the op)."""
    n = rowptr.shape[0] - 1
    rows = torch.repeat_interleave(torch.arange(n, device=rowptr.device), rowptr[1:] - rowptr[:-1])
    want = beta * Y0.double()
    want.index_add_(0, rows, vals.double()[:, None] * X.double()[colidx.long()])
    return want


def _symbol():
    from spcomm3d_b200.utils import native
    lib = native.cuda()
    fn = lib.sp3_cuda_spmm_f32_noalloc
    c = ctypes
    fn.restype = c.c_int
    fn.argtypes = [c.c_int, c.c_int, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_longlong,
                   c.c_int, c.c_float, c.c_void_p, c.c_longlong, c.c_void_p, c.c_void_p, c.c_int, c.c_int,
                   c.c_int, c.c_void_p]
    return fn


def _call(fn, rowptr, colidx, vals, X, Y, beta, sched, total_pieces=None):
    return fn(rowptr.shape[0] - 1, sched.items.shape[0], sched.items.data_ptr(), rowptr.data_ptr(),
              colidx.data_ptr(), vals.data_ptr(), X.data_ptr(), X.stride(0), X.shape[1], beta, Y.data_ptr(),
              Y.stride(0), sched.first.data_ptr(), sched.npieces.data_ptr(), sched.nlong,
              sched.total_pieces if total_pieces is None else total_pieces, sched.piece_len,
              torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("k", [64, 128])
def test_noalloc_matches_regular_entry_point_twice(k):
    from spcomm3d_b200.ops import cuda_ops
    fn = _symbol()
    for call, (seed, beta) in enumerate([(1, 0.0), (2, 0.5)]):
        rowptr, colidx, vals, X, Y0 = _problem(seed, k)
        sched = cuda_ops.SpmmSchedule(rowptr)
        assert sched.nlong == 4
        _compare(fn, rowptr, colidx, vals, X, Y0, beta, sched, call)


def _copy_keeping_ld(t):
    """A copy of a 2-D tensor with the same leading dimension (clone() would pack a column slice)."""
    wide = torch.empty(t.shape[0], t.stride(0), dtype=t.dtype, device=t.device)
    out = wide[:, :t.shape[1]]
    out.copy_(t)
    return out


def _compare(fn, rowptr, colidx, vals, X, Y0, beta, sched, call=0):
    from spcomm3d_b200.ops import cuda_ops
    want = _copy_keeping_ld(Y0)
    cuda_ops.spmm(rowptr, None, colidx, vals, X, want, beta, sched)
    got = _copy_keeping_ld(Y0)
    assert got.stride(0) == Y0.stride(0)
    rc = _call(fn, rowptr, colidx, vals, X, got, beta, sched)
    torch.cuda.synchronize()
    assert rc == 0, f"call {call} returned {rc}"
    # same kernel, same piece order: identical up to the tolerance of the fp32 kernel tests
    assert (got - want).abs().max().item() <= 2e-5 * want.abs().max().item()
    # and both agree with the fp64 result of the same product
    ref = _fp64(rowptr, colidx, vals, X, Y0, beta)
    assert (got.double() - ref).abs().max().item() <= 2e-5 * ref.abs().max().item() * 8


@pytest.mark.parametrize("k,long_rows,ld", [(64, (), None),       # no split rows: the scratch is not touched
                                            (30, (700,), None),   # k not a multiple of 4: scalar kernel
                                            (64, (600, 1500), 96)])  # X and Y are views with ld > k
def test_noalloc_other_shapes_twice(k, long_rows, ld):
    from spcomm3d_b200.ops import cuda_ops
    fn = _symbol()
    for call, (seed, beta) in enumerate([(4, 0.0), (5, -1.0)]):
        rowptr, colidx, vals, X, Y0 = _problem(seed, k, long_rows, ld)
        sched = cuda_ops.SpmmSchedule(rowptr)
        assert sched.nlong == len(long_rows)
        _compare(fn, rowptr, colidx, vals, X, Y0, beta, sched, call)


def test_noalloc_rejects_what_does_not_fit():
    from spcomm3d_b200.ops import cuda_ops
    fn = _symbol()
    rowptr, colidx, vals, X, Y0 = _problem(3, 64)
    sched = cuda_ops.SpmmSchedule(rowptr)
    before = Y0.clone()
    rc = _call(fn, rowptr, colidx, vals, X, Y0, 0.0, sched, total_pieces=10_000_000)
    torch.cuda.synchronize()
    assert rc == -5
    assert torch.equal(Y0, before)  # nothing was launched
