"""Sampled correctness check of a distributed SDDMM + SpMM step.

Dense operands of the benchmarks are pure functions of (seed, stream, global
row, global column) (`utils.generate.fill_rows`), so every rank can rebuild,
in fp64 on the host, the exact inputs of any result entry it owns without
communication: a few thousand owned SDDMM values and a few hundred owned SpMM
rows are recomputed and compared.  A wrong gather (missed or misplaced remote
row), a lost partial result or a broken reduction along the Z fiber changes
these values by O(1); rounding in fp32 changes them by about 1e-6.

The reference's own check compares one global sum of SDDMM values by eye and
has none for SpMM (miniapp/numResCheck_sddmm_parallel.cpp:181-195).
"""
from __future__ import annotations

import numpy as np
import torch

from ..utils import generate


def sample_sddmm_error(plan, c_owned: torch.Tensor, k: int, seed: int, stream_a: int, stream_b: int,
                       n_samples: int = 4096, rng_seed: int = 0, positions=None) -> float:
    """max |C - C_ref| / max |C_ref| over a sample of this rank's slice of C
    (full-k dot products: the Z reduction has already summed the k slices).
    `positions[i]` = position in the plan's CSR order of c_owned[i]
    (`DistSDDMM.owned_positions()`; default: the rank's contiguous CSR slice)."""
    off, length = plan.owned_nnz_slice()
    if length == 0:
        return 0.0
    rng = np.random.default_rng(rng_seed + 7919 * plan.rank)
    idx = np.sort(rng.choice(length, size=min(n_samples, length), replace=False))
    pos = off + idx if positions is None else np.asarray(positions)[idx]
    grow = plan.row.local_gids[plan.rowidx[pos]]
    gcol = plan.col.local_gids[plan.colidx[pos]]
    A = generate.fill_rows(grow, k, 0, k, seed=seed, stream=stream_a, dtype=np.float64)
    B = generate.fill_rows(gcol, k, 0, k, seed=seed, stream=stream_b, dtype=np.float64)
    ref = plan.vals[pos] * np.einsum("ij,ij->i", A, B)
    got = c_owned[torch.from_numpy(idx).to(c_owned.device)].double().cpu().numpy()
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def sample_spmm_error(plan, m, y_owned: torch.Tensor, k: int, seed: int, stream_x: int,
                      n_rows: int = 256, max_nnz: int = 1 << 20, rng_seed: int = 0) -> float:
    """max |Y - Y_ref| / max |Y_ref| over a sample of this rank's owned rows of
    Y = S X, my k slice.  `m` is the whole matrix (global ids), or a function
    that returns all entries of given global rows: a row of Y sums over all
    mesh columns, not only this rank's block."""
    n_owned = plan.row.n_owned
    if n_owned == 0:
        return 0.0
    k_off, k_loc = plan.k_slice(k)
    rng = np.random.default_rng(rng_seed + 104729 * plan.rank)
    loc = np.sort(rng.choice(n_owned, size=min(n_rows, n_owned), replace=False))
    gids = plan.row.owned_gids[loc]
    if callable(m):
        m = m(gids)
    sel = np.flatnonzero(np.isin(m.rows, gids.astype(m.rows.dtype)))
    if sel.size > max_nnz:  # a hub row was drawn: keep whole rows up to the limit
        order = np.argsort(m.rows[sel], kind="stable")
        sel = sel[order]
        deg = np.bincount(np.searchsorted(gids, m.rows[sel]), minlength=gids.size)
        keep_rows = np.cumsum(deg) <= max_nnz
        keep_rows[0] = True
        gids, loc = gids[keep_rows], loc[keep_rows]
        sel = sel[np.isin(m.rows[sel], gids.astype(m.rows.dtype))]
    r = np.searchsorted(gids, m.rows[sel])
    ucols, inv = np.unique(m.cols[sel], return_inverse=True)
    X = generate.fill_rows(ucols, k, k_off, k_loc, seed=seed, stream=stream_x, dtype=np.float64)
    ref = np.zeros((gids.size, k_loc))
    np.add.at(ref, r, m.vals[sel][:, None] * X[inv])
    got = y_owned[torch.from_numpy(loc).to(y_owned.device)].double().cpu().numpy()
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))
