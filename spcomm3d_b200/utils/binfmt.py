"""The conv2bin binary matrix format and the MatrixMarket reader.

Format (verified against the reference writer tools/read_convert_mm.cpp:81-94):
little-endian `u32 nrows, u32 ncols, u64 nnz` followed by nnz 16-byte records
`{u32 row, u32 col, f64 val}`, 0-based, in source order.  The parsing and
writing run in the native host library (csrc/host/io.cpp).
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import native
from .sparse import CooMatrix


def _name_of(path: str) -> str:
    # basename without extension, as the reference derives mtxName
    # (miniapp/bench_spmm.cpp:133-135)
    return os.path.splitext(os.path.basename(path))[0]


def read_bin_header(path: str):
    nr, nc, nnz = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint64()
    rc = native.host().sp3_bin_read_header(path.encode(), ctypes.addressof(nr), ctypes.addressof(nc),
                                           ctypes.addressof(nnz))
    native.check(rc, f"read header of {path}")
    return nr.value, nc.value, nnz.value


def read_bin(path: str, start: int = 0, count: int | None = None) -> CooMatrix:
    """Reads triplets [start, start+count) (default: all) of a .bin file."""
    nr, nc, nnz = read_bin_header(path)
    if count is None:
        count = nnz - start
    rows = np.empty(count, np.uint32)
    cols = np.empty(count, np.uint32)
    vals = np.empty(count, np.float64)
    rc = native.host().sp3_bin_read_range(path.encode(), start, count, native.ptr(rows), native.ptr(cols),
                                          native.ptr(vals), None)
    native.check(rc, f"read {path}")
    return CooMatrix(nr, nc, rows, cols, vals, name=_name_of(path))


def chunk_range(nnz: int, nparts: int, part: int):
    """Contiguous slice of the nnz records read by `part` out of `nparts`
    readers: the first nnz % nparts readers take one extra record
    (src/parallel_io.hpp:81-90)."""
    base, rem = divmod(nnz, nparts)
    start = part * base + min(part, rem)
    return start, base + (1 if part < rem else 0)


def write_bin(path: str, m: CooMatrix):
    rc = native.host().sp3_bin_write(path.encode(), m.nrows, m.ncols, m.nnz, native.ptr(m.rows),
                                     native.ptr(m.cols), native.ptr(m.vals), None)
    native.check(rc, f"write {path}")


def read_mtx(path: str, mirror_diagonal: bool = True) -> CooMatrix:
    """MatrixMarket coordinate file -> CooMatrix.

    pattern -> value 1.0, complex -> real part, symmetric -> expanded.  With
    `mirror_diagonal=True` (default) diagonal entries of symmetric files are
    mirrored too, exactly as the reference does (src/mm.hpp:32,53-57), so the
    resulting .bin is byte-identical to the reference's conv2bin; pass False
    to store each diagonal entry once.
    """
    h = native.host()
    nr, nc, fnnz, cap = (ctypes.c_uint64() for _ in range(4))
    flags = ctypes.c_int()
    rc = h.sp3_mm_read_header(path.encode(), *(ctypes.addressof(v) for v in (nr, nc, fnnz, cap)),
                              ctypes.addressof(flags))
    native.check(rc, f"read header of {path}")
    rows = np.empty(cap.value, np.uint32)
    cols = np.empty(cap.value, np.uint32)
    vals = np.empty(cap.value, np.float64)
    got = ctypes.c_uint64()
    rc = h.sp3_mm_read(path.encode(), cap.value, int(mirror_diagonal), native.ptr(rows), native.ptr(cols),
                       native.ptr(vals), ctypes.addressof(got))
    native.check(rc, f"read {path}")
    n = got.value
    return CooMatrix(nr.value, nc.value, rows[:n], cols[:n], vals[:n], name=_name_of(path))


def write_mtx(path: str, m: CooMatrix):
    rc = native.host().sp3_mm_write(path.encode(), m.nrows, m.ncols, m.nnz, native.ptr(m.rows),
                                    native.ptr(m.cols), native.ptr(m.vals))
    native.check(rc, f"write {path}")


def conv2bin(mtx_path: str, out_path: str | None = None, mirror_diagonal: bool = True) -> str:
    """mtx -> bin; default output name swaps the extension for `.bin`
    (tools/read_convert_mm.cpp:124-126)."""
    if out_path is None:
        out_path = os.path.splitext(mtx_path)[0] + ".bin"
    write_bin(out_path, read_mtx(mtx_path, mirror_diagonal))
    return out_path
