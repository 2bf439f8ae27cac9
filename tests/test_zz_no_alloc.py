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


def _problem(seed, k):
    rng = np.random.default_rng(seed)
    nrows, ncols = 2000, 1500
    deg = rng.poisson(5, nrows)
    deg[rng.integers(0, nrows, 4)] = [600, 1100, 2100, 513]
    rowptr = torch.zeros(nrows + 1, dtype=torch.int64)
    rowptr[1:] = torch.from_numpy(np.cumsum(deg))
    nnz = int(rowptr[-1])
    colidx = torch.from_numpy(rng.integers(0, ncols, nnz).astype(np.int32))
    vals = torch.from_numpy(rng.random(nnz).astype(np.float32))
    X = torch.from_numpy(rng.standard_normal((ncols, k)).astype(np.float32))
    Y0 = torch.from_numpy(rng.standard_normal((nrows, k)).astype(np.float32))
    return rowptr.cuda(), colidx.cuda(), vals.cuda(), X.cuda(), Y0.cuda()


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
        want = Y0.clone()
        cuda_ops.spmm(rowptr, None, colidx, vals, X, want, beta, sched)
        got = Y0.clone()
        rc = _call(fn, rowptr, colidx, vals, X, got, beta, sched)
        torch.cuda.synchronize()
        assert rc == 0, f"call {call} returned {rc}"
        # same kernel, same piece order: identical up to the tolerance of the fp32 kernel tests
        assert (got - want).abs().max().item() <= 2e-5 * want.abs().max().item()


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
