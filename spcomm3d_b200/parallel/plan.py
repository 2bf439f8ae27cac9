"""Sparsity-aware communication plans.

A `SidePlan` describes, for one rank and one side of the sparse block (the
row side: A / Y rows, peers along the mesh row; the column side: B / X rows,
peers along the mesh column), exactly which dense rows the rank owns, needs
and must serve:

* local dense layout `[owned rows (ascending global id) | rows needed from
  peer 0 | from peer 1 | ...]`, each peer's group ascending by global id
  (the reference's receive-in-place layout, src/comm_setup.cpp:373-381);
* per needed row: owning peer and index inside the owner's owned block, which
  is all a pulling kernel needs (`peer_base[owner] + index * ld`);
* per peer: the owned rows that peer needs (send list), which the packed
  NCCL path and the SpMM reduce at the owner need.

`RankPlan` = row SidePlan + column SidePlan + the local block in CSR order
with indices rewritten to the local layouts (localizeIndices + ReMapIndices,
src/SparseMatrix.hpp:69-106) + the slice of nonzero values this rank owns
after the Z reduction (src/comm_setup.cpp:671-689).

The communication volume of a plan is by construction the sparsity-aware
minimum: every needed, non-owned row appears exactly once.  Builders in the
reference: src/comm_setup.cpp:20-140 (one side), :300-432 (receive in
place), :434-577 (both sides in one handle), :759-786 (SpMM: expand X,
reversed expand for Y).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from ..utils import native
from ..utils.sparse import CooMatrix
from .mesh import Mesh3D, split_k, split_nnz
from .partition import Directory


@dataclass
class SidePlan:
    side: str                  # "row" (A/Y, peers vary in y) or "col" (B/X, peers vary in x)
    npeers: int                # length of the mesh line (Y for rows, X for cols)
    me: int                    # my coordinate along that line
    owned_gids: np.ndarray     # int64 [n_owned] ascending
    local_gids: np.ndarray     # int64 [n_local] = owned ++ needed (grouped by owner)
    recv_counts: np.ndarray    # int64 [npeers] rows needed from each peer (0 for me)
    recv_src_idx: np.ndarray   # int32 [n_local - n_owned] index in the owner's owned block
    recv_peer: np.ndarray      # int32 [n_local - n_owned] owning peer of each needed row
    send_counts: np.ndarray    # int64 [npeers] rows each peer needs from me
    send_idx: np.ndarray       # int64 [sum send_counts] my owned-local indices, peer by peer
    peer_owned: np.ndarray     # int64 [npeers] size of every peer's owned block
    push_offset: np.ndarray = None  # int64 [npeers] where my rows start inside peer p's send list

    @property
    def n_owned(self) -> int:
        return int(self.owned_gids.shape[0])

    @property
    def n_local(self) -> int:
        return int(self.local_gids.shape[0])

    @property
    def n_recv(self) -> int:
        return self.n_local - self.n_owned

    @property
    def n_send(self) -> int:
        return int(self.send_idx.shape[0])

    def recv_offsets(self):
        return np.concatenate([[0], np.cumsum(self.recv_counts)])

    def send_offsets(self):
        return np.concatenate([[0], np.cumsum(self.send_counts)])

    def in_degree(self) -> int:
        return int((self.recv_counts > 0).sum())

    def out_degree(self) -> int:
        return int((self.send_counts > 0).sum())


def build_side(directory: Directory, side: str, x: int, y: int) -> SidePlan:
    d = directory
    if side == "row":
        linemap, mask, owner, pos, line, me, npeers = d.rowmap, d.row_mask, d.row_owner, d.row_pos, x, y, d.mesh.Y
        counts = d.row_counts[x]
    else:
        linemap, mask, owner, pos, line, me, npeers = d.colmap, d.col_mask, d.col_owner, d.col_pos, y, x, d.mesh.X
        counts = d.col_counts[y]
    in_line = np.flatnonzero(linemap == line)
    own = owner[in_line] == me
    lmask = mask[in_line]
    touched = ((lmask >> me) & 1).astype(bool)
    owned_gids = in_line[own]
    need = in_line[touched & ~own]
    need_owner = owner[need]
    order = np.argsort(need_owner, kind="stable")
    need, need_owner = need[order], need_owner[order]
    recv_counts = np.bincount(need_owner, minlength=npeers).astype(np.int64)
    send_counts = np.zeros(npeers, np.int64)
    send_parts = []
    own_mask = lmask[own]
    own_pos = pos[owned_gids].astype(np.int64)
    for p in range(npeers):
        if p == me:
            continue
        sel = ((own_mask >> p) & 1).astype(bool)
        send_parts.append(own_pos[sel])
        send_counts[p] = int(sel.sum())
    send_idx = np.concatenate(send_parts) if send_parts else np.zeros(0, np.int64)
    # cnt[q, p] = rows owned by p that q needs; peer p's send list is ordered by q, so my segment in it
    # starts after the segments of all q < me
    line_owner = owner[in_line]
    cnt = np.zeros((npeers, npeers), np.int64)
    for q in range(npeers):
        cnt[q] = np.bincount(line_owner[((lmask >> q) & 1).astype(bool)], minlength=npeers)
        cnt[q, q] = 0
    push_offset = cnt[:me].sum(axis=0)
    return SidePlan(side, npeers, me, owned_gids.astype(np.int64),
                    np.concatenate([owned_gids, need]).astype(np.int64), recv_counts,
                    pos[need].astype(np.int32), need_owner.astype(np.int32), send_counts,
                    send_idx.astype(np.int64), np.asarray(counts, np.int64).copy(), push_offset)


@dataclass
class RankPlan:
    mesh: Mesh3D
    coords: tuple              # (x, y, z)
    nrows: int                 # global dims
    ncols: int
    name: str
    row: SidePlan
    col: SidePlan
    rowptr: np.ndarray         # int64 [row.n_local + 1]
    rowidx: np.ndarray         # int32 [nnz] local row of each nonzero (CSR order)
    colidx: np.ndarray         # int32 [nnz] local column
    vals: np.ndarray           # float64 [nnz]
    src_perm: np.ndarray       # int64 [nnz] position in the block's source order
    gnnz: int = 0              # nonzeros of the whole matrix (for GFLOP/s)
    meta: dict = field(default_factory=dict)

    @property
    def nnz(self) -> int:
        return int(self.colidx.shape[0])

    @property
    def rank(self) -> int:
        return self.mesh.rank_of(*self.coords)

    def k_slice(self, k: int):
        return split_k(k, self.mesh.Z, self.coords[2])

    def owned_nnz_slice(self):
        """(offset, length) of the CSR-ordered values this rank owns after the
        Z reduction of SDDMM."""
        return split_nnz(self.nnz, self.mesh.Z, self.coords[2])

    def global_rows(self) -> np.ndarray:
        return self.row.local_gids[self.rowidx]

    def global_cols(self) -> np.ndarray:
        return self.col.local_gids[self.colidx]

    # ---- volumes, in dense rows (multiply by k_loc for elements) ----------
    def expand_rows(self, sides=("row", "col")):
        """(send_rows, recv_rows, send_msgs, recv_msgs) of the pre-communication."""
        s = r = sm = rm = 0
        for name in sides:
            sp = getattr(self, name)
            s += sp.n_send
            r += sp.n_recv
            sm += sp.out_degree()
            rm += sp.in_degree()
        return s, r, sm, rm

    def validate(self):
        rp, cp = self.row, self.col
        assert self.rowptr.shape[0] == rp.n_local + 1 and self.rowptr[-1] == self.nnz
        if self.nnz:
            assert 0 <= self.rowidx.min() and self.rowidx.max() < rp.n_local
            assert 0 <= self.colidx.min() and self.colidx.max() < cp.n_local
            assert np.all(np.diff(self.rowidx) >= 0)
        for sp in (rp, cp):
            assert sp.recv_counts[sp.me] == 0 and sp.send_counts[sp.me] == 0
            assert sp.recv_counts.sum() == sp.n_recv
            if sp.n_recv:
                assert np.all(sp.recv_src_idx < sp.peer_owned[sp.recv_peer])
            if sp.n_send:
                assert sp.send_idx.max() < sp.n_owned
        return self

    # ---- persistence: plans are reusable across k and across runs ---------
    def save(self, path: str):
        arrays = {"rowptr": self.rowptr, "rowidx": self.rowidx, "colidx": self.colidx, "vals": self.vals,
                  "src_perm": self.src_perm}
        for name in ("row", "col"):
            sp = getattr(self, name)
            for f in ("owned_gids", "local_gids", "recv_counts", "recv_src_idx", "recv_peer", "send_counts",
                      "send_idx", "peer_owned", "push_offset"):
                arrays[f"{name}.{f}"] = getattr(sp, f)
        hdr = np.array([self.mesh.X, self.mesh.Y, self.mesh.Z, *self.coords, self.nrows, self.ncols, self.gnnz,
                        self.row.npeers, self.row.me, self.col.npeers, self.col.me], np.int64)
        np.savez(path, header=hdr, name=np.array(self.name), **arrays)

    @staticmethod
    def load(path: str) -> "RankPlan":
        z = np.load(path if path.endswith(".npz") else path + ".npz")
        h = z["header"]
        mesh = Mesh3D(int(h[0]), int(h[1]), int(h[2]))
        sides = {}
        for name, npeers, me in (("row", int(h[9]), int(h[10])), ("col", int(h[11]), int(h[12]))):
            sides[name] = SidePlan(name, npeers, me, *(z[f"{name}.{f}"] for f in (
                "owned_gids", "local_gids", "recv_counts", "recv_src_idx", "recv_peer", "send_counts",
                "send_idx", "peer_owned", "push_offset")))
        return RankPlan(mesh, (int(h[3]), int(h[4]), int(h[5])), int(h[6]), int(h[7]), str(z["name"]),
                        sides["row"], sides["col"], z["rowptr"], z["rowidx"], z["colidx"], z["vals"],
                        z["src_perm"], gnnz=int(h[8]))


def build_rank_plan(block: CooMatrix, directory: Directory, coords, gnnz: int | None = None) -> RankPlan:
    """Plan of rank `coords` from its block (global ids) and the directory."""
    x, y, z = coords
    rp = build_side(directory, "row", x, y)
    cp = build_side(directory, "col", x, y)
    h = native.host()
    # global -> local tables (the gtlR/gtlC hash maps of SparseMatrix.hpp:26-27, as flat arrays)
    g2l_r = np.full(directory.nrows, -1, np.int32)
    g2l_r[rp.local_gids] = np.arange(rp.n_local, dtype=np.int32)
    g2l_c = np.full(directory.ncols, -1, np.int32)
    g2l_c[cp.local_gids] = np.arange(cp.n_local, dtype=np.int32)
    lrow = np.empty(block.nnz, np.int32)
    lcol = np.empty(block.nnz, np.int32)
    native.check(h.sp3_remap_u32(block.nnz, native.ptr(block.rows), native.ptr(g2l_r), directory.nrows,
                                 native.ptr(lrow)), "localize rows (block holds a row outside its plan)")
    native.check(h.sp3_remap_u32(block.nnz, native.ptr(block.cols), native.ptr(g2l_c), directory.ncols,
                                 native.ptr(lcol)), "localize cols (block holds a column outside its plan)")
    rowptr = np.empty(rp.n_local + 1, np.int64)
    perm = np.empty(block.nnz, np.int64)
    native.check(h.sp3_csr_order(block.nnz, native.ptr(lrow), native.ptr(lcol), rp.n_local, native.ptr(rowptr),
                                 native.ptr(perm)), "csr order")
    return RankPlan(directory.mesh, (x, y, z), directory.nrows, directory.ncols, block.name, rp, cp, rowptr,
                    lrow[perm], lcol[perm], block.vals[perm], perm,
                    gnnz=block.nnz if gnnz is None else gnnz)


def build_all_plans(m: CooMatrix, mesh: Mesh3D, seed: int = 0, policy: str = "respect_comm",
                    z_layers=None):
    """Virtual-mesh builder: plans of every rank in one process (S is
    replicated along Z, so the z layers of one (x, y) share arrays).
    Returns (directory, {rank: RankPlan})."""
    from .partition import bucket_blocks, extract_block
    directory = Directory.from_global(m, mesh, seed, policy)
    offsets, perm = bucket_blocks(m, directory.rowmap, directory.colmap, mesh)
    plans = {}
    zs = range(mesh.Z) if z_layers is None else z_layers
    for x in range(mesh.X):
        for y in range(mesh.Y):
            blk = extract_block(m, offsets, perm, mesh, x, y)
            base = build_rank_plan(blk, directory, (x, y, 0), gnnz=m.nnz)
            for z in zs:
                p = RankPlan(mesh, (x, y, z), base.nrows, base.ncols, base.name, base.row, base.col,
                             base.rowptr, base.rowidx, base.colidx, base.vals, base.src_perm, gnnz=m.nnz)
                plans[mesh.rank_of(x, y, z)] = p
    return directory, plans


def build_my_plan(m: CooMatrix, mesh: Mesh3D, rank: int, seed: int = 0, policy: str = "respect_comm",
                  directory: Directory | None = None):
    """Plan of one rank when every rank holds (or can generate) the full
    matrix: no communication at all."""
    from .partition import bucket_blocks, extract_block
    if directory is None:
        directory = Directory.from_global(m, mesh, seed, policy)
    x, y, z = mesh.coords_of(rank)
    offsets, perm = bucket_blocks(m, directory.rowmap, directory.colmap, mesh)
    blk = extract_block(m, offsets, perm, mesh, x, y)
    return directory, build_rank_plan(blk, directory, (x, y, z), gnnz=m.nnz)


def build_my_plan_from_spec(spec: str, mesh: Mesh3D, groups, seed: int = 0, policy: str = "respect_comm"):
    """Plan of the calling rank for a synthetic matrix, with every rank generating only its own block where the
    generator allows it (uniform, zipf, er): the 2D maps are functions of the seed, the block is generated in
    place, and the touch masks are summed over the plane (the one collective of setup).  Other generators fall
    back to building the whole matrix on every rank.  Returns (directory, plan, whole matrix or None)."""
    from ..utils import generate
    from .partition import directory_from_blocks, make_maps
    rank = groups.rank if groups is not None else 0
    x, y, z = mesh.coords_of(rank)
    if groups is not None and mesh.size > 1:
        probe = generate._spec_rowptr(spec, seed)
        if probe is not None:
            nrows, ncols = probe[0], probe[1]
            rowmap, colmap = make_maps(nrows, ncols, mesh, seed)
            block, gnnz = generate.block_from_spec(spec, seed, rowmap, x, colmap, y)
            directory = directory_from_blocks(block, mesh, groups, seed, rowmap, colmap, policy)
            return directory, build_rank_plan(block, directory, (x, y, z), gnnz=gnnz), None
    m = generate.from_spec(spec, seed=seed)
    directory, plan = build_my_plan(m, mesh, rank, seed=seed, policy=policy)
    return directory, plan, m
