"""Dense-panel SDDMM and SpMM: tensor-core tiles where the nonzeros are dense enough.

`PanelSDDMM` splits the nonzeros of a CSR block (local indices) into

* panels -- (128-row block, up to 64 columns) pairs in which every chosen
  column holds at least `min_col_nnz` nonzeros of the block; each panel is one
  128 x 64 x k TF32 product on the tcgen05 tensor cores
  (csrc/kernels/panel_ops.cu), sampled at the nonzero positions; and
* the remainder, which runs through the regular gather kernel with its results
  scattered to their positions in the value array.

`PanelSpMM` uses the same split: all panels of a 128-row block accumulate
`S_panel (128 x 64) @ X[panel columns] (64 x k)` in one TMEM tile that is added
to the Y rows of the block after the gather kernel has handled the remainder.

TF32 rounds the operands to 10 mantissa bits, so panel values carry a relative
error of about 1e-3 of |A row| * |B row| (SpMM: of sum |s| * |x|); the path is
opt-in.  The reference has one scalar loop per kernel (src/core_ops.cpp:5-35).
"""
from __future__ import annotations

import numpy as np
import torch

from ..utils import native
from . import cuda_ops

PANEL_M, PANEL_N = 128, 64


class PanelSDDMM:
    def __init__(self, rowidx: np.ndarray, colidx: np.ndarray, vals: np.ndarray, nrows_a: int, ncols_b: int,
                 device="cuda", min_col_nnz: int = 3, min_panel_nnz: int = 192):
        dev = torch.device(device)
        nnz = rowidx.shape[0]
        self.nnz, self.nrows_a = nnz, nrows_a
        blk = rowidx.astype(np.int64) // PANEL_M
        key = blk * ncols_b + colidx.astype(np.int64)
        uniq, inv, cnt = np.unique(key, return_inverse=True, return_counts=True)
        dense = cnt >= min_col_nnz
        pair_blk = uniq // ncols_b
        # slot of every dense (block, column) pair inside its block, in column order
        didx = np.flatnonzero(dense)
        first = np.searchsorted(pair_blk[didx], pair_blk[didx], side="left")
        slot = np.arange(didx.size) - first
        pair_panel_local = slot // PANEL_N           # tile number inside the block
        # global panel id per dense pair
        pkey = pair_blk[didx] * (1 << 20) + pair_panel_local
        pu, pinv = np.unique(pkey, return_inverse=True)
        pair_panel = np.full(uniq.size, -1, np.int64)
        pair_panel[didx] = pinv
        pair_slot = np.zeros(uniq.size, np.int64)
        pair_slot[didx] = slot % PANEL_N
        e_panel = pair_panel[inv]
        # drop thin panels
        pn = np.bincount(e_panel[e_panel >= 0], minlength=pu.size)
        keep = pn >= min_panel_nnz
        renum = np.cumsum(keep) - 1
        in_panel = (e_panel >= 0) & keep[np.maximum(e_panel, 0)]
        self.npanels = int(keep.sum())
        sel = np.flatnonzero(in_panel)
        order = sel[np.argsort(renum[e_panel[sel]], kind="stable")]
        ep = renum[e_panel[order]]
        ptr = np.zeros(self.npanels + 1, np.int64)
        np.cumsum(np.bincount(ep, minlength=self.npanels), out=ptr[1:])
        cols = np.zeros((max(self.npanels, 1), PANEL_N), np.int32)
        kp = np.flatnonzero(keep[pinv])  # dense pairs of kept panels
        cols[renum[pinv[kp]], slot[kp] % PANEL_N] = (uniq[didx[kp]] % ncols_b).astype(np.int32)
        row0 = np.zeros(max(self.npanels, 1), np.int32)
        row0[renum[pinv[kp]]] = (pair_blk[didx[kp]] * PANEL_M).astype(np.int32)
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a.astype(dt))).to(dev)
        self.panel_row0, self.panel_cols, self.panel_ptr = t(row0, np.int32), t(cols, np.int32), t(ptr, np.int32)
        self.e_row = t(rowidx[order] - blk[order] * PANEL_M, np.uint8)
        self.e_col = t(pair_slot[inv[order]], np.uint8)
        self.e_pos = t(order, np.int32)
        self.e_sval = t(vals[order], np.float32)
        rest = np.flatnonzero(~in_panel)
        self.n_panel_nnz, self.n_rest = int(order.size), int(rest.size)
        self.r_row, self.r_col = t(rowidx[rest], np.int32), t(colidx[rest], np.int32)
        self.r_val, self.r_pos = t(vals[rest], np.float32), t(rest, np.int32)
        self.status = cuda_ops.new_status(dev)

    def run(self, A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(self.nnz, dtype=torch.float32, device=A.device)
        lib, st = native.cuda(), torch.cuda.current_stream().cuda_stream
        k = A.shape[1]
        if self.npanels:
            rc = lib.sp3_cuda_sddmm_panel_f32(self.npanels, native.ptr(self.panel_row0), native.ptr(self.panel_cols),
                                              native.ptr(self.panel_ptr), native.ptr(self.e_row), native.ptr(self.e_col),
                                              native.ptr(self.e_pos), native.ptr(self.e_sval), native.ptr(A),
                                              A.stride(0), self.nrows_a, native.ptr(B), B.stride(0), k,
                                              native.ptr(out), native.ptr(self.status), st)
            if rc == -1:
                raise ValueError("panel kernel needs fp32, k a multiple of 8 and at most 128")
            cuda_ops._ck(rc, "sddmm_panel")
        if self.n_rest:
            rc = lib.sp3_cuda_sddmm_orig_f32(self.n_rest, native.ptr(self.r_row), native.ptr(self.r_col),
                                             native.ptr(self.r_val), native.ptr(A), A.stride(0), native.ptr(B),
                                             B.stride(0), k, native.ptr(out), native.ptr(self.r_pos), st)
            cuda_ops._ck(rc, "sddmm remainder")
        return out


class PanelSpMM:
    """Y = beta * Y + S @ X with the dense panels of S on the tensor cores.

    rowidx must be sorted ascending (CSR order of the local block)."""

    def __init__(self, rowidx: np.ndarray, colidx: np.ndarray, vals: np.ndarray, nrows_y: int, ncols_x: int,
                 device="cuda", min_col_nnz: int = 3, min_panel_nnz: int = 192, group_panels: int = 8):
        self.split = s = PanelSDDMM(rowidx, colidx, vals, nrows_y, ncols_x, device, min_col_nnz, min_panel_nnz)
        self.nrows_y, self.npanels, self.n_panel_nnz, self.n_rest = nrows_y, s.npanels, s.n_panel_nnz, s.n_rest
        dev = torch.device(device)
        # Panels are numbered block by block.  Up to `group_panels` consecutive panels of one row block form a
        # group (one accumulator tile, one CTA); a hub block with more panels is cut into several groups, which
        # then add to the same Y rows atomically.
        r0 = s.panel_row0.cpu().numpy()[:s.npanels]
        if s.npanels:
            first = np.flatnonzero(np.r_[True, r0[1:] != r0[:-1]])
            blk_of = np.cumsum(np.r_[True, r0[1:] != r0[:-1]]) - 1
            within = np.arange(s.npanels) - first[blk_of]
            # at most 16 groups per row block: more would only queue up on the atomic adds to the same rows
            n_in_blk = np.bincount(blk_of)
            gsize = np.maximum(group_panels, -(-n_in_blk // 16))[blk_of]
            starts = np.flatnonzero(within % gsize == 0)
            per_blk = np.bincount(blk_of[starts])
            shared = (per_blk[blk_of[starts]] > 1).astype(np.uint8)
        else:
            starts, shared = np.zeros(0, np.int64), np.zeros(0, np.uint8)
        self.ngroups = int(starts.size)
        self.grp_ptr = torch.from_numpy(np.r_[starts, s.npanels].astype(np.int32)).to(dev)
        self.grp_shared = torch.from_numpy(np.r_[shared, np.uint8(0)].astype(np.uint8)).to(dev)
        # remainder as CSR over all rows, with its own schedule
        rr = s.r_row.cpu().numpy()
        if rr.size and np.any(rr[1:] < rr[:-1]):
            raise ValueError("PanelSpMM needs row-sorted nonzeros")
        rp = np.zeros(nrows_y + 1, np.int64)
        np.cumsum(np.bincount(rr, minlength=nrows_y), out=rp[1:])
        self.rowptr = torch.from_numpy(rp).to(dev)
        self.sched = cuda_ops.SpmmSchedule(self.rowptr)
        self.status = s.status

    def run(self, X: torch.Tensor, Y: torch.Tensor, beta: float = 0.0) -> torch.Tensor:
        s = self.split
        k = X.shape[1]
        if k % 32 or k > 256:
            raise ValueError("SpMM panel kernel needs fp32 and k a multiple of 32, at most 256")
        cuda_ops.spmm(self.rowptr, s.r_row, s.r_col, s.r_val, X, Y, beta, self.sched)
        if self.ngroups:
            lib, st = native.cuda(), torch.cuda.current_stream().cuda_stream
            rc = lib.sp3_cuda_spmm_panel_f32(self.ngroups, native.ptr(self.grp_ptr), native.ptr(self.grp_shared),
                                             native.ptr(s.panel_row0),
                                             native.ptr(s.panel_cols), native.ptr(s.panel_ptr), native.ptr(s.e_row),
                                             native.ptr(s.e_col), native.ptr(s.e_sval), native.ptr(X), X.stride(0), k,
                                             native.ptr(Y), Y.stride(0), self.nrows_y, native.ptr(self.status), st)
            if rc == -1:
                raise ValueError("SpMM panel kernel: unsupported shape or alignment")
            cuda_ops._ck(rc, "spmm_panel")
        return Y
