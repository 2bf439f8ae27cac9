"""Single-process fp64 oracles in plain PyTorch.

`sddmm_ref`:  C[i] = S.val[i] * <A[S.row[i], :], B[S.col[i], :]>
`spmm_ref`:   Y[r, :] = beta*Y[r, :] + sum_{(r,c,v) in S} v * X[c, :]

These restate the reference loops src/core_ops.cpp:5-35 with vectorised
tensor ops and are what every kernel and every distributed path is compared
against.  `checksum` is the scalar the reference checkers print
(miniapp/numCheckSeq.cpp:130-132).
"""
from __future__ import annotations

import numpy as np
import torch

from ..utils.sparse import CooMatrix


def _t(x, dtype=torch.float64):
    if isinstance(x, np.ndarray):
        x = torch.from_numpy(x)
    return x.to(dtype=dtype, device="cpu")


def sddmm_ref(m: CooMatrix, A, B, chunk: int = 1 << 20) -> torch.Tensor:
    A, B = _t(A), _t(B)
    r = torch.from_numpy(m.rows.astype(np.int64))
    c = torch.from_numpy(m.cols.astype(np.int64))
    v = torch.from_numpy(m.vals)
    out = torch.empty(m.nnz, dtype=torch.float64)
    for s in range(0, m.nnz, chunk):
        e = min(m.nnz, s + chunk)
        out[s:e] = (A[r[s:e]] * B[c[s:e]]).sum(dim=1) * v[s:e]
    return out


def spmm_ref(m: CooMatrix, X, Y=None, beta: float = 0.0) -> torch.Tensor:
    X = _t(X)
    out = torch.zeros(m.nrows, X.shape[1], dtype=torch.float64) if Y is None or beta == 0.0 else _t(Y) * beta
    r = torch.from_numpy(m.rows.astype(np.int64))
    c = torch.from_numpy(m.cols.astype(np.int64))
    v = torch.from_numpy(m.vals)
    chunk = 1 << 20
    for s in range(0, m.nnz, chunk):
        e = min(m.nnz, s + chunk)
        out.index_add_(0, r[s:e], X[c[s:e]] * v[s:e, None])
    return out


def checksum(values) -> float:
    return float(_t(values).sum())
