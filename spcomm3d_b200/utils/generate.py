"""Seeded synthetic matrices and dense operands.

Generators for the benchmark families: fixed-degree uniform, R-MAT,
Zipf-row-degree rectangular and Erdos-Renyi.  All randomness is counter based
(csrc/host/generate.cpp), so a spec string + seed names one matrix everywhere.
The reference has only an unseeded unique-position generator
(src/SparseMatrix.hpp:49-67).
"""
from __future__ import annotations

import numpy as np

from . import native
from .sparse import CooMatrix


def fixed_degree(nrows: int, ncols: int, degree: int, seed: int = 0) -> CooMatrix:
    """`degree` distinct uniform columns in every row, values U(0,1)."""
    nnz = nrows * degree
    rows, cols, vals = np.empty(nnz, np.uint32), np.empty(nnz, np.uint32), np.empty(nnz, np.float64)
    rc = native.host().sp3_gen_fixed_degree(nrows, ncols, degree, seed, native.ptr(rows), native.ptr(cols),
                                            native.ptr(vals))
    native.check(rc, "fixed_degree generator")
    return CooMatrix(nrows, ncols, rows, cols, vals, name=f"uniform_{nrows}x{ncols}_d{degree}")


def _from_degrees(nrows, ncols, deg, seed, name) -> CooMatrix:
    rowptr = np.zeros(nrows + 1, np.uint64)
    np.cumsum(deg, out=rowptr[1:])
    nnz = int(rowptr[-1])
    rows, cols, vals = np.empty(nnz, np.uint32), np.empty(nnz, np.uint32), np.empty(nnz, np.float64)
    rc = native.host().sp3_gen_from_rowptr(nrows, ncols, native.ptr(rowptr), seed, native.ptr(rows),
                                           native.ptr(cols), native.ptr(vals))
    native.check(rc, f"{name} generator")
    return CooMatrix(nrows, ncols, rows, cols, vals, name=name)


def zipf_rows(nrows: int, ncols: int, alpha: float = 1.8, dmin: int = 1, dmax: int = 4096,
              seed: int = 0) -> CooMatrix:
    """Row degrees follow a power law P(d >= x) = x^-(alpha-1) clipped to
    [dmin, dmax]; columns uniform without replacement; values U(0,1)."""
    deg = np.empty(nrows, np.uint32)
    rc = native.host().sp3_gen_degrees(nrows, 0, alpha, dmin, min(dmax, ncols), seed, native.ptr(deg))
    native.check(rc, "zipf degrees")
    return _from_degrees(nrows, ncols, deg, seed, f"zipf_{nrows}x{ncols}_a{alpha}")


def erdos_renyi(nrows: int, ncols: int, mean_degree: float, seed: int = 0) -> CooMatrix:
    """Every position present with probability mean_degree/ncols: row degrees
    are Poisson(mean_degree), columns uniform; values U(0,1)."""
    deg = np.empty(nrows, np.uint32)
    rc = native.host().sp3_gen_degrees(nrows, 1, float(mean_degree), 0, ncols, seed, native.ptr(deg))
    native.check(rc, "poisson degrees")
    return _from_degrees(nrows, ncols, deg, seed, f"er_{nrows}x{ncols}_d{mean_degree:g}")


def rmat(scale: int, edge_factor: int = 16, a: float = 0.57, b: float = 0.19, c: float = 0.19,
         seed: int = 0) -> CooMatrix:
    """R-MAT graph with 2^scale vertices and edge_factor * 2^scale drawn edges,
    duplicates removed, values U(0,1); entries sorted by (row, col)."""
    n = 1 << scale
    m = edge_factor * n
    keys = np.empty(m, np.uint64)
    h = native.host()
    native.check(h.sp3_gen_rmat_keys(scale, m, a, b, c, seed, native.ptr(keys)), "rmat generator")
    nu = h.sp3_sort_unique_u64(native.ptr(keys), m)
    rows, cols, vals = np.empty(nu, np.uint32), np.empty(nu, np.uint32), np.empty(nu, np.float64)
    native.check(h.sp3_keys_to_coo(native.ptr(keys), nu, seed, native.ptr(rows), native.ptr(cols),
                                   native.ptr(vals)), "rmat split")
    return CooMatrix(n, n, rows, cols, vals, name=f"rmat_s{scale}_ef{edge_factor}")


def random_nnz(nrows: int, ncols: int, nnz: int, seed: int = 0) -> CooMatrix:
    """Exactly `nnz` distinct positions drawn uniformly, every value 1.0, sorted by (row, col)
    (`CooMatrix.random_unique`; the reference's COOMatrix::self_generate_random, src/SparseMatrix.hpp:49-67)."""
    m = CooMatrix.random_unique(nrows, ncols, nnz, seed)
    m.name = f"random_{nrows}x{ncols}_nnz{nnz}"
    return m


def from_spec(spec: str, seed: int = 0) -> CooMatrix:
    """Parses `uniform:M:N:deg`, `rmat:scale[:ef]`, `zipf:M:N[:alpha[:dmax]]`,
    `er:M:N:mean_degree`, `random:M:N:nnz`."""
    kind, *args = spec.split(":")
    if kind == "random":
        return random_nnz(int(args[0]), int(args[1]), int(args[2]), seed)
    if kind == "uniform":
        return fixed_degree(int(args[0]), int(args[1]), int(args[2]), seed)
    if kind == "rmat":
        return rmat(int(args[0]), int(args[1]) if len(args) > 1 else 16, seed=seed)
    if kind == "zipf":
        return zipf_rows(int(args[0]), int(args[1]), float(args[2]) if len(args) > 2 else 1.8,
                         dmax=int(args[3]) if len(args) > 3 else 4096, seed=seed)
    if kind == "er":
        return erdos_renyi(int(args[0]), int(args[1]), float(args[2]), seed)
    raise ValueError(f"unknown generator spec {spec!r}")


def _spec_rowptr(spec: str, seed: int):
    """(nrows, ncols, rowptr, name) for the generators that draw every row independently (uniform, zipf, er);
    None for the others (rmat removes duplicates globally, random draws positions globally)."""
    kind, *args = spec.split(":")
    h = native.host()
    if kind == "uniform":
        nrows, ncols, d = int(args[0]), int(args[1]), int(args[2])
        deg = np.full(nrows, d, np.uint32)
        name = f"uniform_{nrows}x{ncols}_d{d}"
    elif kind == "zipf":
        nrows, ncols = int(args[0]), int(args[1])
        alpha = float(args[2]) if len(args) > 2 else 1.8
        dmax = int(args[3]) if len(args) > 3 else 4096
        deg = np.empty(nrows, np.uint32)
        native.check(h.sp3_gen_degrees(nrows, 0, alpha, 1, min(dmax, ncols), seed, native.ptr(deg)), "zipf degrees")
        name = f"zipf_{nrows}x{ncols}_a{alpha}"
    elif kind == "er":
        nrows, ncols, mean = int(args[0]), int(args[1]), float(args[2])
        deg = np.empty(nrows, np.uint32)
        native.check(h.sp3_gen_degrees(nrows, 1, mean, 0, ncols, seed, native.ptr(deg)), "poisson degrees")
        name = f"er_{nrows}x{ncols}_d{mean:g}"
    else:
        return None
    rowptr = np.zeros(nrows + 1, np.uint64)
    np.cumsum(deg, out=rowptr[1:])
    return nrows, ncols, rowptr, name


def block_from_spec(spec: str, seed: int, rowmap=None, x: int = 0, colmap=None, y: int = 0):
    """The part of the matrix `from_spec(spec, seed)` that lies in rows with rowmap == x and columns with
    colmap == y (None keeps a whole side), generated directly: entry for entry the same positions and values as
    in the whole matrix, without ever building it.  Returns (block with global ids, nonzeros of the whole
    matrix), or None for generators that cannot be restricted (rmat, random).  This is what lets every rank
    build only its own block of a synthetic matrix; the reference reads its chunk of a file instead
    (src/parallel_io.hpp:81-127)."""
    got = _spec_rowptr(spec, seed)
    if got is None:
        return None
    nrows, ncols, rowptr, name = got
    rm = None if rowmap is None else np.ascontiguousarray(rowmap, dtype=np.int32)
    cm = None if colmap is None else np.ascontiguousarray(colmap, dtype=np.int32)
    import ctypes
    cnt = ctypes.c_uint64()
    fn = native.host().sp3_gen_from_rowptr_block
    native.check(fn(nrows, ncols, native.ptr(rowptr), seed, native.ptr(rm), x, native.ptr(cm), y,
                    ctypes.addressof(cnt), None, None, None), f"{name} block count")
    n = int(cnt.value)
    rows, cols, vals = np.empty(n, np.uint32), np.empty(n, np.uint32), np.empty(n, np.float64)
    native.check(fn(nrows, ncols, native.ptr(rowptr), seed, native.ptr(rm), x, native.ptr(cm), y,
                    ctypes.addressof(cnt), native.ptr(rows), native.ptr(cols), native.ptr(vals)), f"{name} block")
    return CooMatrix(nrows, ncols, rows, cols, vals, name=name), int(rowptr[-1])


def rows_from_spec(spec: str, seed: int, row_ids):
    """All entries of the given rows of `from_spec(spec, seed)` (the others are never generated), or None."""
    got = _spec_rowptr(spec, seed)
    if got is None:
        return None
    sel = np.ones(got[0], np.int32)
    sel[np.asarray(row_ids, dtype=np.int64)] = 0
    return block_from_spec(spec, seed, rowmap=sel, x=0)[0]


FILL_NORMAL, FILL_GID_OVER_1000, FILL_CONST = 0, 1, 2


def fill_rows(gids, k_global: int, col0: int, ncols: int, *, kind: int = FILL_NORMAL, const: float = 0.0,
              seed: int = 0, stream: int = 0, dtype=np.float32, ld: int | None = None) -> np.ndarray:
    """Rows `gids` and columns [col0, col0+ncols) of a virtual global dense
    matrix with k_global columns whose entries are a pure function of
    (seed, stream, global row, global column).  kind: N(0,1), gid/1000 (the
    fill used by the reference checkers, miniapp/numCheckSeq.cpp:125-128), or a
    constant."""
    gids = np.ascontiguousarray(gids, dtype=np.int64)
    ld = ncols if ld is None else ld
    out = np.zeros((gids.shape[0], ld), dtype=dtype)
    fn = native.host().sp3_fill_rows_f32 if dtype == np.float32 else native.host().sp3_fill_rows_f64
    rc = fn(native.ptr(gids), gids.shape[0], col0, ncols, ld, k_global, kind, const, seed, stream,
            native.ptr(out))
    native.check(rc, "fill_rows")
    return out
