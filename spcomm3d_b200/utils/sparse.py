"""Host-side sparse containers.

`CooMatrix` is the framework's interchange form of a (global or local) sparse
matrix: parallel arrays of u32 row ids, u32 column ids and f64 values, like the
reference's COOMatrix `ii/jj/vv` (src/SparseMatrix.hpp:12-41) but as numpy
arrays, without the per-matrix hash maps.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class CooMatrix:
    nrows: int
    ncols: int
    rows: np.ndarray  # uint32 [nnz]
    cols: np.ndarray  # uint32 [nnz]
    vals: np.ndarray  # float64 [nnz]
    name: str = "matrix"

    def __post_init__(self):
        self.rows = np.ascontiguousarray(self.rows, dtype=np.uint32)
        self.cols = np.ascontiguousarray(self.cols, dtype=np.uint32)
        self.vals = np.ascontiguousarray(self.vals, dtype=np.float64)
        if not (len(self.rows) == len(self.cols) == len(self.vals)):
            raise ValueError("rows/cols/vals lengths differ")

    @property
    def nnz(self) -> int:
        return int(self.rows.shape[0])

    @property
    def shape(self):
        return (self.nrows, self.ncols)

    def validate(self):
        if self.nnz:
            if int(self.rows.max()) >= self.nrows or int(self.cols.max()) >= self.ncols:
                raise ValueError("index out of range")
        return self

    def to_torch_sparse(self, dtype=None):
        import torch
        idx = torch.from_numpy(np.stack([self.rows.astype(np.int64), self.cols.astype(np.int64)]))
        v = torch.from_numpy(self.vals)
        if dtype is not None:
            v = v.to(dtype)
        return torch.sparse_coo_tensor(idx, v, (self.nrows, self.ncols))

    def random_unique(nrows: int, ncols: int, nnz: int, seed: int = 0) -> "CooMatrix":
        """nnz distinct positions, value 1.0: the seeded counterpart of the
        reference's `self_generate_random` (src/SparseMatrix.hpp:49-67)."""
        rng = np.random.default_rng(seed)
        if nnz > nrows * ncols:
            raise ValueError("more nonzeros than positions")
        keys = np.unique(rng.integers(0, nrows * ncols, size=int(nnz * 1.2) + 16, dtype=np.int64))
        while keys.size < nnz:
            keys = np.unique(np.concatenate([keys, rng.integers(0, nrows * ncols, size=nnz, dtype=np.int64)]))
        keys = np.sort(rng.permutation(keys)[:nnz])
        return CooMatrix(nrows, ncols, keys // ncols, keys % ncols, np.ones(nnz), name="random")

    random_unique = staticmethod(random_unique)
