"""Python front end of the local sm_100a kernels (csrc/kernels/local_ops.cu).

Every function launches on the current torch CUDA stream and passes raw device
pointers; nothing here falls back to a torch implementation.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..utils import native

_F = {torch.float32: "f32", torch.float64: "f64"}

# SpMM schedule parameters: rows with more than LONG_ROW nonzeros are cut into
# pieces of LONG_ROW; other rows are grouped into items of about ITEM_NNZ
# nonzeros and at most ITEM_ROWS rows.
LONG_ROW = int(os.environ.get("SP3_LONG_ROW", 512))
ITEM_NNZ = int(os.environ.get("SP3_ITEM_NNZ", 128))
ITEM_ROWS = int(os.environ.get("SP3_ITEM_ROWS", 64))


PIECE_SHIFT = 20   # SPMM_PIECE_SHIFT of csrc/kernels/sp3_kernels.cuh


def _stream():
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = 0  # kernels launched through this module (bench.py reports the count)


def _ck(rc, what, n=1):
    global LAUNCHES
    LAUNCHES += n
    if rc != 0:
        raise RuntimeError(f"{what}: CUDA launch error {rc}")


def _ld(t):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("dense operand must be 2-D with unit inner stride")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


USE_TMA = os.environ.get("SP3_SDDMM_TMA", "0") == "1"


def sddmm_tma(rowidx, colidx, svals, A, B, out, status=None):
    """SDDMM whose B rows are staged in shared memory by TMA `tile::gather4`
    copies (csrc/kernels/tma_ops.cu).  fp32, k a multiple of 8 in [8, 256]."""
    if A.dtype != torch.float32:
        raise TypeError("the TMA kernel is fp32")
    st = new_status(A.device) if status is None else status
    rc = native.cuda().sp3_cuda_sddmm_tma_f32(rowidx.shape[0], native.ptr(rowidx), native.ptr(colidx),
                                              native.ptr(svals), native.ptr(A), _ld(A), native.ptr(B), _ld(B),
                                              B.shape[0], A.shape[1], native.ptr(out), native.ptr(st), _stream())
    if rc < 0:
        raise ValueError({-1: "shape not supported by the TMA kernel", -2: "tensor map encoding failed"}[rc])
    _ck(rc, "sddmm_tma")
    return out


def sddmm(rowidx, colidx, svals, A, B, out):
    if USE_TMA and A.dtype == torch.float32 and A.shape[1] % 8 == 0 and 8 <= A.shape[1] <= 256:
        return sddmm_tma(rowidx, colidx, svals, A, B, out)
    fn = getattr(native.cuda(), f"sp3_cuda_sddmm_{_F[A.dtype]}")
    _ck(fn(rowidx.shape[0], native.ptr(rowidx), native.ptr(colidx), native.ptr(svals), native.ptr(A), _ld(A),
           native.ptr(B), _ld(B), A.shape[1], native.ptr(out), _stream()), "sddmm")
    return out


def build_spmm_items(rowptr: np.ndarray, long_row: int | None = None, item_nnz: int | None = None,
                     item_rows: int | None = None):
    """Work items of the SpMM kernel from a CSR row pointer (host, vectorised).

    Returns (items int32[n,4], first_piece int32[nlong], npieces int32[nlong]).
    rows item  = (row_begin, row_end, 0, -1)
    piece item = (row, nnz_begin, nnz_end, long_row_slot | piece_number_in_row << PIECE_SHIFT)
    """
    long_row = LONG_ROW if long_row is None else long_row
    item_nnz = ITEM_NNZ if item_nnz is None else item_nnz
    item_rows = ITEM_ROWS if item_rows is None else item_rows
    nrows = rowptr.shape[0] - 1
    deg = np.diff(rowptr)
    is_long = deg > long_row
    key = rowptr[:-1] // item_nnz
    bnd = np.ones(nrows, bool)
    if nrows > 1:
        bnd[1:] = (key[1:] != key[:-1]) | (np.arange(1, nrows) % item_rows == 0) | is_long[1:] | is_long[:-1]
    starts = np.flatnonzero(bnd)
    ends = np.append(starts[1:], nrows)
    short = ~is_long[starts]
    rows_items = np.stack([starts[short], ends[short], np.zeros(short.sum(), np.int64),
                           -np.ones(short.sum(), np.int64)], axis=1)
    long_rows = np.flatnonzero(is_long)
    npieces = (deg[long_rows] + long_row - 1) // long_row
    first = np.concatenate([[0], np.cumsum(npieces)[:-1]]) if long_rows.size else np.zeros(0, np.int64)
    if long_rows.size:
        slot = np.repeat(np.arange(long_rows.size), npieces)
        j = np.arange(int(npieces.sum())) - np.repeat(first, npieces)
        r = long_rows[slot]
        b = rowptr[r] + j * long_row
        e = np.minimum(b + long_row, rowptr[r + 1])
        if long_rows.size >= 1 << PIECE_SHIFT or int(npieces.max()) >= 1 << (31 - PIECE_SHIFT):
            raise ValueError("too many split rows or pieces per row for the item encoding")
        piece_items = np.stack([r, b, e, slot + (j << PIECE_SHIFT)], axis=1)
        items = np.concatenate([piece_items, rows_items])  # heavy work first
    else:
        items = rows_items
    if items.size and items.max() >= 2 ** 31:
        raise ValueError("more than 2^31 nonzeros or rows on one rank")
    return items.astype(np.int32), first.astype(np.int32), npieces.astype(np.int32)


def build_spmm_wave_items(rowptr: np.ndarray, cls: np.ndarray, n_classes: int, long_row: int | None = None,
                          item_nnz: int | None = None, item_rows: int | None = None):
    """Work items for an SpMM whose column-side rows arrive in waves.  `cls[q]` is the class of nonzero q
    (0: its dense row is there from the start; c: it arrives with wave c - 1).

    Long rows have their nonzeros sorted by class (stable) and are cut into pieces at class boundaries (and
    every `long_row` nonzeros), so that the part of a hub row whose columns are already there is computable at
    once; other rows are grouped as in `build_spmm_items` and take the largest class of their nonzeros.  Items
    are returned sorted by class.

    Returns (perm int64[nnz]: source position of every nonzero of the re-ordered CSR arrays, items, first_piece,
    npieces, class_items int32[n_classes]: number of items of classes 0..c)."""
    long_row = LONG_ROW if long_row is None else long_row
    nnz = int(rowptr[-1])
    deg = np.diff(rowptr)
    std_items, _, _ = build_spmm_items(rowptr, long_row, item_nnz, item_rows)
    rows_items = std_items[std_items[:, 3] < 0].astype(np.int64)
    perm = np.arange(nnz, dtype=np.int64)
    lrows = np.flatnonzero(deg > long_row)
    pieces = np.zeros((0, 4), np.int64)
    pcls = np.zeros(0, np.int64)
    first = np.zeros(0, np.int64)
    npieces = np.zeros(0, np.int64)
    if lrows.size >= 1 << PIECE_SHIFT:
        raise ValueError("too many split rows for the item encoding")
    if lrows.size:
        ldeg = deg[lrows]
        lstart = np.cumsum(ldeg) - ldeg                        # first position of every long row in `idx`
        slot_of = np.repeat(np.arange(lrows.size, dtype=np.int32), ldeg)
        idx = np.arange(int(ldeg.sum()), dtype=np.int64)
        idx += np.repeat(rowptr[lrows] - lstart, ldeg)         # nonzeros of the long rows, ascending
        key = slot_of * np.int32(256)                          # < 2^28: the slot count is checked below
        key += cls[idx]
        order = np.argsort(key, kind="stable")
        src = idx[order]
        perm[idx] = src
        key = key[order]                                       # slot_of is already grouped by row
        c_sorted = key & np.int32(255)
        # runs of equal (row, class), cut every long_row nonzeros
        run_start = np.flatnonzero(np.concatenate([[True], key[1:] != key[:-1]]))
        run_len = np.diff(np.append(run_start, key.size))
        nchunk = (run_len + long_row - 1) // long_row
        chunk_run = np.repeat(np.arange(run_start.size), nchunk)
        chunk_j = np.arange(int(nchunk.sum())) - np.repeat(np.cumsum(nchunk) - nchunk, nchunk)
        b_rel = run_start[chunk_run] + chunk_j * long_row
        e_rel = np.minimum(b_rel + long_row, run_start[chunk_run] + run_len[chunk_run])
        p_slot = slot_of[b_rel]
        npieces = np.bincount(p_slot, minlength=lrows.size)
        first = np.cumsum(npieces) - npieces
        p_num = np.arange(p_slot.size) - first[p_slot]
        if int(npieces.max()) >= 1 << (31 - PIECE_SHIFT):
            raise ValueError("too many pieces per row for the item encoding")
        pieces = np.stack([lrows[p_slot], idx[b_rel], idx[b_rel] + (e_rel - b_rel), p_slot + (p_num << PIECE_SHIFT)], axis=1)
        pcls = c_sorted[b_rel].astype(np.int64)
    # class of a rows item: the largest class among its nonzeros
    rcls = np.zeros(rows_items.shape[0], np.int64)
    if rows_items.shape[0] and nnz:
        b, e = rowptr[rows_items[:, 0]], rowptr[rows_items[:, 1]]
        nonempty = e > b
        if nonempty.any():
            cmax = np.maximum.reduceat(np.append(cls, cls.dtype.type(0)), np.stack([b[nonempty], e[nonempty]], 1).ravel())[::2]
            rcls[nonempty] = cmax
    items = np.concatenate([pieces, rows_items])
    icls = np.concatenate([pcls, rcls])
    order = np.argsort(icls, kind="stable")                    # pieces stay ahead of rows items inside a class
    items = items[order]
    class_items = np.cumsum(np.bincount(icls, minlength=n_classes))[:n_classes]
    if items.size and items.max() >= 2 ** 31:
        raise ValueError("more than 2^31 nonzeros or rows on one rank")
    return perm, items.astype(np.int32), first.astype(np.int32), npieces.astype(np.int32), class_items.astype(np.int32)


class SpmmSchedule:
    """Device-resident SpMM work items plus the scratch the long-row path
    needs: one carry row per piece and one counter per long row."""

    def __init__(self, rowptr: torch.Tensor, k_max: int = 0, dtype=torch.float32, arrays=None, **kw):
        if arrays is None:
            rp = rowptr.cpu().numpy()
            items, first, npieces = build_spmm_items(rp, **kw)
        else:   # (items, first_piece, npieces) built elsewhere, e.g. by build_spmm_wave_items
            items, first, npieces = arrays
        dev = rowptr.device
        self.piece_len = kw.get("long_row", LONG_ROW)
        self.items = torch.from_numpy(items).to(dev).contiguous()
        self.first = torch.from_numpy(first).to(dev)
        self.npieces = torch.from_numpy(npieces).to(dev)
        self.counters = torch.zeros(max(1, first.shape[0]), dtype=torch.int32, device=dev)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        self.total_pieces = int(npieces.sum())
        self.carry = None
        self.nlong = int(first.shape[0])

    def carry_for(self, k: int, dtype, device):
        if self.total_pieces == 0:
            return None, 0
        if self.carry is None or self.carry.shape[1] < k or self.carry.dtype != dtype:
            self.carry = torch.empty(self.total_pieces, k, dtype=dtype, device=device)
        return self.carry, self.carry.stride(0)


USE_SPMM_TMA = os.environ.get("SP3_SPMM_TMA", "0") == "1"


def spmm_tma(rowidx, colidx, vals, X, Y, beta=0.0, status=None):
    """SpMM whose X rows are staged in shared memory by TMA `tile::gather4`
    copies (csrc/kernels/tma_ops.cu).  rowidx ascending (CSR order), fp32, k a
    multiple of 8 in [8, 256].  Rows that span several 256-nonzero units are
    summed with atomics (not bitwise reproducible)."""
    if X.dtype != torch.float32:
        raise TypeError("the TMA kernel is fp32")
    st = new_status(X.device) if status is None else status
    rc = native.cuda().sp3_cuda_spmm_tma_f32(rowidx.shape[0], native.ptr(rowidx), native.ptr(colidx), native.ptr(vals),
                                             native.ptr(X), _ld(X), X.shape[0], X.shape[1], float(beta),
                                             native.ptr(Y), _ld(Y), Y.shape[0], native.ptr(st), _stream())
    if rc < 0:
        raise ValueError({-1: "shape not supported by the TMA kernel", -2: "tensor map encoding failed"}[rc])
    _ck(rc, "spmm_tma", 2)
    return Y


def spmm(rowptr, rowidx, colidx, vals, X, Y, beta, sched: SpmmSchedule | None):
    if USE_SPMM_TMA and X.dtype == torch.float32 and X.shape[1] % 8 == 0 and 8 <= X.shape[1] <= 256:
        return spmm_tma(rowidx, colidx, vals, X, Y, beta)
    if sched is None:
        sched = SpmmSchedule(rowptr)
    carry, ldc = sched.carry_for(X.shape[1], X.dtype, X.device)
    fn = getattr(native.cuda(), f"sp3_cuda_spmm_{_F[X.dtype]}")
    _ck(fn(rowptr.shape[0] - 1, sched.items.shape[0], native.ptr(sched.items), native.ptr(rowptr),
           native.ptr(colidx), native.ptr(vals), native.ptr(X), _ld(X), X.shape[1], float(beta), native.ptr(Y),
           _ld(Y), native.ptr(sched.first), native.ptr(sched.npieces), native.ptr(sched.counters),
           native.ptr(carry), ldc, sched.piece_len, native.ptr(sched.ticket), _stream()), "spmm")
    return Y


def rows(mode, idx, src, dst):
    fn = getattr(native.cuda(), f"sp3_cuda_rows_{_F[src.dtype]}")
    _ck(fn(mode, idx.shape[0], native.ptr(idx), native.ptr(src), _ld(src), native.ptr(dst), _ld(dst),
           src.shape[1], _stream()), "rows")
    return dst


def fill_rows(gids: torch.Tensor, k_global, col0, out: torch.Tensor, *, kind=0, const=0.0, seed=0, stream=0):
    """Device twin of utils.generate.fill_rows: writes into out[len(gids), ncols]."""
    fn = getattr(native.cuda(), f"sp3_cuda_fill_rows_{_F[out.dtype]}")
    _ck(fn(native.ptr(gids), gids.shape[0], col0, out.shape[1], _ld(out), k_global, kind, float(const), seed,
           stream, native.ptr(out), _stream()), "fill_rows")
    return out


def checksum(x: torch.Tensor) -> torch.Tensor:
    """fp64 sum of a 1-D fp32/fp64 tensor with a fixed reduction shape."""
    part = torch.empty(1024, dtype=torch.float64, device=x.device)
    out = torch.empty(1, dtype=torch.float64, device=x.device)
    fn = getattr(native.cuda(), f"sp3_cuda_sum_{_F[x.dtype]}")
    _ck(fn(native.ptr(x), x.numel(), native.ptr(part), native.ptr(out), _stream()), "checksum", 2)
    return out


def new_status(device):
    return torch.zeros(4, dtype=torch.int32, device=device)


def validate_indices(rowidx: torch.Tensor, colidx: torch.Tensor, nrows: int, ncols: int):
    """Debug aid (the role compute-sanitizer would play): checks on the device
    that all local row / column indices are in range and raises with the first
    offender instead of letting a kernel read out of bounds."""
    st = new_status(rowidx.device)
    lib = native.cuda()
    _ck(lib.sp3_cuda_check_range(rowidx.shape[0], native.ptr(rowidx), nrows, 0, native.ptr(st), _stream()), "check rows")
    _ck(lib.sp3_cuda_check_range(colidx.shape[0], native.ptr(colidx), ncols, 1, native.ptr(st), _stream()), "check cols")
    code, which, pos, val = st.tolist()
    if code:
        raise IndexError(f"{'row' if which == 0 else 'column'} index {val} at nonzero {pos} is outside "
                         f"[0, {nrows if which == 0 else ncols})")


def remap_indices(idx: torch.Tensor, table: torch.Tensor, status=None) -> torch.Tensor:
    out = torch.empty_like(idx)
    st = new_status(idx.device) if status is None else status
    _ck(native.cuda().sp3_cuda_remap(idx.shape[0], native.ptr(idx), native.ptr(table), table.shape[0],
                                     native.ptr(out), native.ptr(st), _stream()), "remap")
    return out


def invert_perm(perm: torch.Tensor, status=None) -> torch.Tensor:
    inv = torch.empty_like(perm)
    st = new_status(perm.device) if status is None else status
    _ck(native.cuda().sp3_cuda_invert_perm(perm.shape[0], native.ptr(perm), native.ptr(inv), native.ptr(st),
                                           _stream()), "invert_perm")
    return inv


def touch_masks(rows_, cols_, rowmap, colmap, row_mask, col_mask):
    _ck(native.cuda().sp3_cuda_touch_masks(rows_.shape[0], native.ptr(rows_), native.ptr(cols_),
                                           native.ptr(rowmap), native.ptr(colmap), native.ptr(row_mask),
                                           native.ptr(col_mask), _stream()), "touch_masks")
    return row_mask, col_mask
