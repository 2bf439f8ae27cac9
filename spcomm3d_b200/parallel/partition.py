"""2D nonzero partition and dense-row ownership.

`Directory` holds, for every global row and column id, its mesh line
(`rowmap[r] in [0,X)`, `colmap[c] in [0,Y)`), its 64-bit touch mask (which
mesh columns / rows hold a nonzero of it), its owner coordinate and its
position inside the owner's ascending owned list.  Everything a rank needs to
know about who owns, needs and sends which dense row is a pure function of
these vectors, so the only collective at setup time is one sum of the masks.

Reference counterparts: random round-robin 2D maps src/parallel_io.hpp:64-79;
nonzero bucketing :95-127; S replicated along Z :152-167; "respect
communication" ownership src/distribute.cpp:27-209 (owner is always a rank
that touches the row, untouched ids round-robin :135-146); random ownership
:212-247.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..utils import native
from ..utils.sparse import CooMatrix
from .mesh import Mesh3D

MAX_LINE = 62  # touch masks are summed as int64, one bit per mesh coordinate

STREAM_ROWMAP, STREAM_COLMAP, STREAM_ROWOWN, STREAM_COLOWN = 101, 102, 103, 104


def make_maps(nrows: int, ncols: int, mesh: Mesh3D, seed: int):
    """Seeded shuffle + round-robin maps of rows over X and columns over Y."""
    if mesh.X > MAX_LINE or mesh.Y > MAX_LINE:
        raise ValueError(f"mesh lines longer than {MAX_LINE} are not supported by mask-based plans")
    rowmap = np.empty(nrows, np.int32)
    colmap = np.empty(ncols, np.int32)
    h = native.host()
    native.check(h.sp3_rr_map(nrows, mesh.X, seed, STREAM_ROWMAP, native.ptr(rowmap)), "rowmap")
    native.check(h.sp3_rr_map(ncols, mesh.Y, seed, STREAM_COLMAP, native.ptr(colmap)), "colmap")
    return rowmap, colmap


def bucket_blocks(m: CooMatrix, rowmap, colmap, mesh: Mesh3D):
    """(offsets[X*Y+1], perm): nonzeros of xy-block b = x*Y+y are
    perm[offsets[b]:offsets[b+1]], in source order."""
    offsets = np.empty(mesh.xy_size + 1, np.int64)
    perm = np.empty(m.nnz, np.int64)
    rc = native.host().sp3_bucket_blocks(m.nnz, native.ptr(m.rows), native.ptr(m.cols), native.ptr(rowmap),
                                         native.ptr(colmap), mesh.X, mesh.Y, native.ptr(offsets),
                                         native.ptr(perm))
    native.check(rc, "bucket_blocks")
    return offsets, perm


def touch_masks(m: CooMatrix, rowmap, colmap, row_mask=None, col_mask=None):
    """Adds the touch bits of the nonzeros of `m` (whole matrix or one block)."""
    if row_mask is None:
        row_mask = np.zeros(m.nrows, np.int64)
    if col_mask is None:
        col_mask = np.zeros(m.ncols, np.int64)
    rc = native.host().sp3_touch_masks(m.nnz, native.ptr(m.rows), native.ptr(m.cols), native.ptr(rowmap),
                                       native.ptr(colmap), native.ptr(row_mask), native.ptr(col_mask))
    native.check(rc, "touch_masks")
    return row_mask, col_mask


@dataclass
class Directory:
    mesh: Mesh3D
    nrows: int
    ncols: int
    seed: int
    policy: str
    rowmap: np.ndarray     # int32 [nrows]  mesh x of each row
    colmap: np.ndarray     # int32 [ncols]  mesh y of each column
    row_mask: np.ndarray   # int64 [nrows]  bit y: block (rowmap[r], y) has a nonzero in row r
    col_mask: np.ndarray   # int64 [ncols]  bit x: block (x, colmap[c]) has a nonzero in column c
    row_owner: np.ndarray  # int32 [nrows]  mesh y of the owner of A/Y row r (its x is rowmap[r])
    row_pos: np.ndarray    # int32 [nrows]  index of r in its owner's ascending owned list
    col_owner: np.ndarray  # int32 [ncols]  mesh x of the owner of B/X row c (its y is colmap[c])
    col_pos: np.ndarray    # int32 [ncols]
    row_counts: np.ndarray  # int64 [X, Y]  owned A rows per xy rank
    col_counts: np.ndarray  # int64 [Y, X]  owned B rows, indexed [y, x]

    @staticmethod
    def from_masks(mesh, nrows, ncols, seed, rowmap, colmap, row_mask, col_mask,
                   policy: str = "respect_comm") -> "Directory":
        pol = {"respect_comm": 0, "random": 1}[policy]
        h = native.host()
        row_owner, row_pos = np.empty(nrows, np.int32), np.empty(nrows, np.int32)
        col_owner, col_pos = np.empty(ncols, np.int32), np.empty(ncols, np.int32)
        row_counts = np.zeros((mesh.X, mesh.Y), np.int64)
        col_counts = np.zeros((mesh.Y, mesh.X), np.int64)
        native.check(h.sp3_assign_owners(nrows, native.ptr(row_mask), native.ptr(rowmap), mesh.X, mesh.Y, pol,
                                         seed, STREAM_ROWOWN, native.ptr(row_owner), native.ptr(row_pos),
                                         native.ptr(row_counts)), "row owners")
        native.check(h.sp3_assign_owners(ncols, native.ptr(col_mask), native.ptr(colmap), mesh.Y, mesh.X, pol,
                                         seed, STREAM_COLOWN, native.ptr(col_owner), native.ptr(col_pos),
                                         native.ptr(col_counts)), "col owners")
        return Directory(mesh, nrows, ncols, seed, policy, rowmap, colmap, row_mask, col_mask,
                         row_owner, row_pos, col_owner, col_pos, row_counts, col_counts)

    @staticmethod
    def from_global(m: CooMatrix, mesh: Mesh3D, seed: int = 0, policy: str = "respect_comm") -> "Directory":
        """All vectors from a matrix every caller holds in full."""
        rowmap, colmap = make_maps(m.nrows, m.ncols, mesh, seed)
        row_mask, col_mask = touch_masks(m, rowmap, colmap)
        return Directory.from_masks(mesh, m.nrows, m.ncols, seed, rowmap, colmap, row_mask, col_mask, policy)

    # the reference's global owner vectors (rank inside the xy plane), distribute.cpp:154-161
    def rpvec(self) -> np.ndarray:
        return self.rowmap.astype(np.int64) * self.mesh.Y + self.row_owner

    def cpvec(self) -> np.ndarray:
        return self.col_owner.astype(np.int64) * self.mesh.Y + self.colmap

    def check(self):
        """Ownership invariants the reference asserts at distribute.cpp:194-206:
        the owner lies in the mesh line fixed by the 2D partition, and is a
        toucher whenever anybody touches the id."""
        m = self.mesh
        assert self.rowmap.min(initial=0) >= 0 and self.rowmap.max(initial=0) < m.X
        assert self.colmap.min(initial=0) >= 0 and self.colmap.max(initial=0) < m.Y
        assert self.row_owner.max(initial=0) < m.Y and self.col_owner.max(initial=0) < m.X
        if self.policy == "respect_comm":
            t = self.row_mask != 0
            assert np.all((self.row_mask[t] >> self.row_owner[t]) & 1)
            t = self.col_mask != 0
            assert np.all((self.col_mask[t] >> self.col_owner[t]) & 1)
        assert int(self.row_counts.sum()) == self.nrows and int(self.col_counts.sum()) == self.ncols
        return self


def extract_block(m: CooMatrix, offsets, perm, mesh: Mesh3D, x: int, y: int) -> CooMatrix:
    """The nonzeros of block (x, y), global ids, source order."""
    b = mesh.xy_rank(x, y)
    sel = perm[offsets[b]:offsets[b + 1]]
    return CooMatrix(m.nrows, m.ncols, m.rows[sel], m.cols[sel], m.vals[sel], name=m.name)


def distribute_from_file(path: str, mesh: Mesh3D, groups, seed: int = 0, policy: str = "respect_comm"):
    """Collective reader: every xy rank of the z == 0 plane reads a contiguous
    chunk of the .bin file, buckets it by destination block and exchanges the
    buckets with all_to_all; the block is then broadcast down each Z fiber and
    the touch masks are summed over the plane.  Returns (block, directory).

    Same data flow as read_bin_parallel_distribute_coo (src/parallel_io.hpp:
    19-190) with the shuffle seeded and identical on every rank (no Bcast of
    the maps) and one bulk read per rank.
    """
    import torch
    import torch.distributed as dist
    from ..utils import binfmt

    nrows, ncols, gnnz = binfmt.read_bin_header(path)
    rowmap, colmap = make_maps(nrows, ncols, mesh, seed)
    x, y, z = groups.coords
    P = mesh.xy_size
    me = mesh.xy_rank(x, y)
    if z == 0:
        start, cnt = binfmt.chunk_range(gnnz, P, me)
        chunk = binfmt.read_bin(path, start, cnt)
        offsets, perm = bucket_blocks(chunk, rowmap, colmap, mesh)
        send_counts = torch.from_numpy(np.diff(offsets).copy())
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=groups.plane)
        s_split, r_split = send_counts.tolist(), recv_counts.tolist()

        def exchange(arr, dtype):
            out = torch.empty(int(sum(r_split)), dtype=dtype)
            dist.all_to_all_single(out, torch.from_numpy(np.ascontiguousarray(arr[perm])).view(dtype),
                                   r_split, s_split, group=groups.plane)
            return out.numpy()

        rows = exchange(chunk.rows.view(np.int32), torch.int32).view(np.uint32)
        cols = exchange(chunk.cols.view(np.int32), torch.int32).view(np.uint32)
        vals = exchange(chunk.vals, torch.float64)
        n = torch.tensor([rows.shape[0]], dtype=torch.int64)
    else:
        n = torch.zeros(1, dtype=torch.int64)
    if mesh.Z > 1:
        root = mesh.rank_of(x, y, 0)
        dist.broadcast(n, src=root, group=groups.fiber)
        if z != 0:
            rows = np.empty(int(n), np.uint32)
            cols = np.empty(int(n), np.uint32)
            vals = np.empty(int(n), np.float64)
        for arr, dt in ((rows, np.int32), (cols, np.int32), (vals, np.float64)):
            t = torch.from_numpy(arr.view(dt))
            dist.broadcast(t, src=root, group=groups.fiber)
    from ..utils.binfmt import _name_of
    block = CooMatrix(nrows, ncols, rows, cols, vals, name=_name_of(path))
    directory = directory_from_blocks(block, mesh, groups, seed, rowmap, colmap, policy)
    return block, directory


def directory_from_blocks(block: CooMatrix, mesh: Mesh3D, groups, seed, rowmap=None, colmap=None,
                          policy: str = "respect_comm") -> Directory:
    """Directory when each rank only holds its own block: local touch bits,
    one all_reduce(SUM) over the xy plane (bits of different ranks in a mesh
    line are disjoint, so the sum is the union), owners evaluated locally."""
    import torch
    import torch.distributed as dist
    if rowmap is None:
        rowmap, colmap = make_maps(block.nrows, block.ncols, mesh, seed)
    row_mask, col_mask = touch_masks(block, rowmap, colmap)
    if mesh.xy_size > 1:
        for mask in (row_mask, col_mask):
            t = torch.from_numpy(mask)
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=groups.plane)
    return Directory.from_masks(mesh, block.nrows, block.ncols, seed, rowmap, colmap, row_mask, col_mask,
                                policy)
