"""Dense-panel SDDMM: tensor-core tiles where the nonzeros are dense enough.

`PanelSDDMM` splits the nonzeros of a CSR block (local indices) into

* panels -- (128-row block, up to 64 columns) pairs in which every chosen
  column holds at least `min_col_nnz` nonzeros of the block; each panel is one
  128 x 64 x k TF32 product on the tcgen05 tensor cores
  (csrc/kernels/panel_ops.cu), sampled at the nonzero positions; and
* the remainder, which runs through the regular gather kernel with its results
  scattered to their positions in the value array.

TF32 rounds the operands to 10 mantissa bits, so panel values carry a relative
error of about 1e-3 of |A row| * |B row|; the path is opt-in.  The reference
has one scalar loop for everything (src/core_ops.cpp:5-22).
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
