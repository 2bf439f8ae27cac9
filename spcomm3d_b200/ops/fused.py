"""Front end of the fused compute+communication kernels (csrc/kernels/fused_impl.cuh).

`FusedSDDMM` / `FusedSpMM` own the symmetric heap of one distributed op, turn
its plan into the pointer tables the kernel needs (absolute addresses of dense
rows in the owners' heaps, of value buffers along the Z fiber, of partial-row
slots at the row owners) and launch one persistent kernel per run.

These are the product path that replaces the reference's message pipelines
(src/distributed_comp.cpp:17-76, 141-284): no staging buffers, no library
collective; remote rows are loaded, and partial results stored, by the kernel
itself through NVLink peer addresses.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

from ..parallel.symm import IpcFabric, SymmHeap, _align
from ..utils import native
from . import cuda_ops

MAX_RANKS = 64
MAX_WAVES = 32   # pull waves a kernel can track (csrc/kernels/fused_impl.cuh)
F_KINDS = 3
PH_START, PH_MAIN, PH_FINISH = 1, 2, 4
PH_ALL = 7
_SITES = {1: "READY flag of a rank whose memory is read", 2: "local pull counter",
          3: "PART flag (partial results) of a contributing rank", 4: "DONE flag of a reader", 100: "flag"}

P = C.c_void_p


class _Comm(C.Structure):
    _fields_ = [("me", C.c_int), ("epoch", C.c_int), ("phases", C.c_int), ("timeout_ns", C.c_ulonglong),
                ("status", P), ("ctrl", P), ("pad", P), ("peer_pad", P), ("read_from", P), ("readers", P),
                ("push_to", P), ("contrib", P), ("n_read", C.c_int), ("n_readers", C.c_int),
                ("n_push", C.c_int), ("n_contrib", C.c_int), ("stamps", P)]


class _PullConfig(C.Structure):
    _fields_ = [("pullers", C.c_int), ("stage_bytes", C.c_uint), ("tile_rows", C.c_int)]


class _SddmmArgs(C.Structure):
    _fields_ = [("comm", _Comm), ("nnz", C.c_longlong), ("rowidx", P), ("colidx", P), ("sval", P),
                ("a_refs", P), ("a_bases", P), ("world", C.c_int), ("B_loc", P), ("ldb", C.c_longlong), ("n_owned_b", C.c_int),
                ("n_recv_b", C.c_int), ("b_src", P), ("nvec", C.c_int), ("Z", C.c_int), ("my_z", C.c_int),
                ("zbase", C.c_uint), ("zrem", C.c_uint), ("zwidth", C.c_longlong), ("zbuf", P), ("out", P),
                ("part", P), ("direct_push", C.c_int), ("orig", P), ("nnz_free", C.c_longlong), ("work_per_pull", C.c_int),
                ("n_recv_a", C.c_int), ("a_src", P), ("A_stage", P), ("mc_part", P), ("part_stride", C.c_longlong),
                ("pull_order", P), ("n_waves", C.c_int), ("tiles_per_wave", C.c_int), ("wave_nnz", P),
                ("pull", _PullConfig)]


class _SpmmLong(C.Structure):
    _fields_ = [("first_piece", P), ("npieces", P), ("counters", P), ("carry", P), ("ldc", C.c_longlong),
                ("piece_len", C.c_int), ("ticket", P)]


class _SpmmArgs(C.Structure):
    _fields_ = [("comm", _Comm), ("nitems", C.c_int), ("items", P), ("rowptr", P), ("colidx", P), ("val", P),
                ("X_loc", P), ("ldx", C.c_longlong), ("n_owned_x", C.c_int), ("n_recv_x", C.c_int),
                ("x_src", P), ("nvec", C.c_int), ("lg", _SpmmLong), ("n_owned_y", C.c_int), ("n_crows", C.c_int),
                ("crows", P), ("y_dst", P), ("parity_off_v", C.c_longlong), ("Y", P),
                ("ldy", C.c_longlong), ("beta", C.c_double), ("cptr", P), ("cslot", P), ("slots", P),
                ("lds", C.c_longlong), ("atomic", C.c_int), ("red_v4", C.c_int), ("crow_flag", P),
                ("pull", _PullConfig), ("n_waves", C.c_int), ("tiles_per_wave", C.c_int), ("wave_items", P),
                ("pull_order", P)]


_checked_layout = False


def _check_layout():
    global _checked_layout
    if _checked_layout:
        return
    a, b, c = C.c_int(), C.c_int(), C.c_int()
    native.cuda().sp3_fused_struct_sizes(C.byref(a), C.byref(b), C.byref(c))
    if (a.value, b.value, c.value) != (C.sizeof(_SddmmArgs), C.sizeof(_SpmmArgs), C.sizeof(_Comm)):
        raise RuntimeError("argument struct layout differs between Python and the kernel library: "
                           f"{(a.value, b.value, c.value)} vs "
                           f"{(C.sizeof(_SddmmArgs), C.sizeof(_SpmmArgs), C.sizeof(_Comm))}")
    _checked_layout = True


class FusedStatusError(RuntimeError):
    pass


def _esize(dtype) -> int:
    return 8 if dtype == torch.float64 else 4


def _pad4(k: int, dtype=torch.float32) -> int:
    """Leading dimension of the dense blocks of the fused kernels: k rounded up so that a row is a whole number
    of 16-byte vectors (4 fp32 or 2 fp64 values) for any k / Z.  The padding columns are zero and stay zero:
    they add nothing to a dot product and produce zeros in a result row."""
    per = 16 // _esize(dtype)
    return (int(k) + per - 1) // per * per


def _bulk_default(bulk_pull):
    """Pull mode of the fused kernels: True = remote rows travel as `cp.async.bulk` copies issued by one warp
    per block (asynchronous copy unit, staged through shared memory); False = vector loads and stores by the
    pulling warps.  Default from SP3_FUSED_BULK (1 unless set to 0)."""
    if bulk_pull is None:
        return os.environ.get("SP3_FUSED_BULK", "1") == "1"
    return bool(bulk_pull)


def _peer_ranks(plan, side: str):
    """World rank of every peer along a side of the plan's mesh position."""
    x, y, z = plan.coords
    m = plan.mesh
    if side == "row":
        return [m.rank_of(x, j, z) for j in range(m.Y)]
    if side == "col":
        return [m.rank_of(i, y, z) for i in range(m.X)]
    return [m.rank_of(x, y, k) for k in range(m.Z)]


def _tiles_by_peer_distance(side, n_tiles: int, tile_rows: int) -> np.ndarray:
    """Tiles of a side's receive list in the order they are pulled: first the tiles whose rows belong to the
    peer after me on the mesh line, then the next peer, and so on round the line.  In ascending order every
    rank of a line would start at peer 0 and move on together, so that at any time one owner serves all
    readers of the line through its one link while the others sit idle.  (A tile that straddles two peers goes
    with the peer of its first row.)  SP3_FUSED_ROTATE=0 keeps the ascending order."""
    tiles = np.arange(n_tiles, dtype=np.int64)
    if n_tiles == 0 or side.npeers <= 2 or os.environ.get("SP3_FUSED_ROTATE", "1") != "1":
        return tiles
    peer = side.recv_peer[tiles * tile_rows].astype(np.int64)
    return np.argsort((peer - side.me - 1) % side.npeers, kind="stable")


class _FusedBase:
    def __init__(self, op, heap: SymmHeap | None, fabric, timeout_s: float):
        _check_layout()
        self.op, self.plan = op, op.plan
        self.device = op.device
        self.k_loc = op.k_loc
        if op.dtype not in (torch.float32, torch.float64):
            raise ValueError("fused kernels are fp32 or fp64")
        self.dtype, self.es = op.dtype, _esize(op.dtype)
        kmax = 4096 // self.es   # a dense row is at most 256 16-byte vectors
        if self.k_loc == 0 or self.k_loc > kmax:
            raise ValueError(f"fused kernels need 1 <= k/Z <= {kmax} for this value type (got {self.k_loc})")
        if self.plan.mesh.size > MAX_RANKS:
            raise ValueError(f"fused kernels support at most {MAX_RANKS} ranks")
        self.kpad = _pad4(self.k_loc, self.dtype)     # leading dimension of every dense block, slot and carry row
        self.row_bytes = self.kpad * self.es
        self.nvec = self.row_bytes // 16
        if heap is None:
            if fabric is None:
                fabric = IpcFabric(device=self.device)
            heap = fabric.heap(self.region_sizes_for(self.plan, self.k_loc))
        self.heap = heap
        self.rank = self.plan.rank
        self.epoch = 0
        self.timeout_ns = int(timeout_s * 1e9)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.ctrl = torch.zeros(int(native.cuda().sp3_fused_ctrl_words()), dtype=torch.int32, device=self.device)
        self.pad = heap.view("pad", torch.int32, (F_KINDS * MAX_RANKS,))
        self.peer_pad = self._dev_i64([heap.addr("pad", r) for r in range(heap.world)])
        self._keep = []

    def region_sizes_for(self, plan, k_loc):
        return self.region_sizes(plan, k_loc, dtype=self.dtype)

    def _pull_config(self, cfg: _PullConfig):
        """Pull set-up of this op: bulk mode = `SP3_FUSED_PULLERS` warps per block (default 1) with ring stages
        of `SP3_FUSED_STAGE_BYTES` (default 8 KB) and pull tickets of about 64 KB; vector-load mode = tickets
        of 64 rows."""
        if self.bulk_pull:
            cfg.pullers = max(1, min(4, int(os.environ.get("SP3_FUSED_PULLERS", "1"))))
            stage = int(os.environ.get("SP3_FUSED_STAGE_BYTES", "8192")) // 16 * 16
            cfg.stage_bytes = max(stage, self.row_bytes, 1024)
            tile_bytes = int(os.environ.get("SP3_FUSED_TILE_BYTES", "65536"))
            cfg.tile_rows = max(16, min(1024, tile_bytes // self.row_bytes))
        else:
            cfg.pullers, cfg.stage_bytes, cfg.tile_rows = 0, 0, 64
        self.tile_rows = int(cfg.tile_rows)

    def _fn(self, kernel: str):
        return getattr(native.cuda(), f"sp3_fused_{kernel}_{'f64' if self.dtype == torch.float64 else 'f32'}")

    def _dev_i64(self, values):
        return torch.from_numpy(np.asarray(values, dtype=np.int64).reshape(-1)).to(self.device)

    def _dev_i32(self, values):
        return torch.from_numpy(np.asarray(values, dtype=np.int32).reshape(-1)).to(self.device)

    def _fill_comm(self, comm: _Comm, read_from, readers, push_to, contrib):
        lists = []
        for name, ranks in (("read_from", read_from), ("readers", readers), ("push_to", push_to),
                            ("contrib", contrib)):
            t = self._dev_i32(sorted(set(int(r) for r in ranks)) or [0])
            n = len(set(ranks))
            lists.append(t)
            setattr(comm, name, t.data_ptr())
            setattr(comm, {"read_from": "n_read", "readers": "n_readers", "push_to": "n_push",
                           "contrib": "n_contrib"}[name], n)
        self._keep.append(lists)
        comm.me = self.rank
        comm.timeout_ns = self.timeout_ns
        comm.status = self.status.data_ptr()
        comm.ctrl = self.ctrl.data_ptr()
        comm.pad = self.pad.data_ptr()
        comm.peer_pad = self.peer_pad.data_ptr()
        self.stamps = torch.zeros(4, dtype=torch.int64, device=self.device)
        comm.stamps = self.stamps.data_ptr()

    def _side_tables(self, side, region):
        """(addresses of every local row in its owner's heap, addresses of the rows to pull)."""
        h, rb = self.heap, self.row_bytes
        ranks = np.asarray(_peer_ranks(self.plan, side.side), dtype=np.int64)
        base = np.asarray(h.peer_base, dtype=np.int64) + h.offsets[region]
        own = base[self.rank] + np.arange(side.n_owned, dtype=np.int64) * rb
        need = base[ranks[side.recv_peer]] + side.recv_src_idx.astype(np.int64) * rb
        return own, need

    def set_timeout(self, seconds: float):
        self.timeout_ns = int(seconds * 1e9)
        self.args.comm.timeout_ns = self.timeout_ns

    def check(self):
        """Synchronises and raises if the last launches recorded a status."""
        torch.cuda.synchronize(self.device)
        st = self.status.tolist()
        if st[0] != 0:
            self.status.zero_()
            what = {1: "bad index", 2: "wait timed out"}.get(st[0], f"code {st[0]}")
            raise FusedStatusError(f"fused kernel on rank {self.rank}: {what} at {_SITES.get(st[1], st[1])}, "
                                   f"peer/slot {st[2]}, observed {st[3]} (epoch {self.epoch})")

    def phase_ms(self) -> dict:
        """Device timestamps of the last launch (synchronises): time from kernel
        start until all remote rows were pulled, until MAIN finished (compute
        done, partial results pushed and signalled) and until the kernel's
        final handshake."""
        torch.cuda.synchronize(self.device)
        t = self.stamps.tolist()
        return {"pull": max(0, t[1] - t[0]) / 1e6, "main": (t[2] - t[0]) / 1e6, "total": (t[3] - t[0]) / 1e6}

    def _launch(self, fn, phases):
        self.args.comm.phases = phases
        self.args.comm.epoch = self.epoch
        rc = fn(C.byref(self.args), torch.cuda.current_stream(self.device).cuda_stream)
        cuda_ops.LAUNCHES += 1
        if rc != 0:
            raise RuntimeError(f"fused kernel launch failed: CUDA error {rc}")


class FusedSDDMM(_FusedBase):
    @staticmethod
    def region_sizes(plan, k_loc: int, dtype=torch.float32) -> dict:
        es = _esize(dtype)
        rb = _pad4(k_loc, dtype) * es
        Z = plan.mesh.Z
        zwidth = plan.nnz // Z + (1 if plan.nnz % Z else 0)
        return {"pad": F_KINDS * MAX_RANKS * 4, "A": plan.row.n_local * rb, "B": plan.col.n_local * rb,
                "zbuf": 2 * Z * zwidth * es if Z > 1 else 0}

    def __init__(self, op, heap: SymmHeap | None = None, fabric=None, timeout_s: float = 30.0,
                 overlap: bool = True, direct_push: bool | None = None, stage_a: bool | None = None,
                 zreduce: str | None = None, bulk_pull: bool | None = None):
        super().__init__(op, heap, fabric, timeout_s)
        self.bulk_pull = _bulk_default(bulk_pull)
        if zreduce is None:
            zreduce = os.environ.get("SP3_FUSED_ZREDUCE", "push")
        if zreduce not in ("push", "multimem"):
            raise ValueError(f"zreduce must be 'push' or 'multimem', got {zreduce!r}")
        self.zreduce = zreduce
        p, h, k = self.plan, self.heap, self.k_loc
        Z, z = p.mesh.Z, p.coords[2]
        # A block: my owned rows (peers read them in place) followed by room for staged copies of the remote
        # rows I need.  stage_a (default): the needed remote A rows are pulled in bulk like the B rows, many
        # loads in flight per warp; the compute loop then reads local memory only.  stage_a=False reads every
        # remote A row straight from its owner when a work unit first needs it: no staging traffic, but the
        # unit stalls for one NVLink round trip per row change, which costs more than the copy on real links.
        if stage_a is None:
            stage_a = os.environ.get("SP3_FUSED_STAGE_A", "1") == "1"
        self.stage_a = bool(stage_a)
        kp = self.kpad
        self._A_full = h.view("A", self.dtype, (p.row.n_local, kp))   # padded storage, see _pad4
        self._B_full = h.view("B", self.dtype, (p.col.n_local, kp))
        self.A_loc = self._A_full[:p.row.n_owned, :k]
        self.B_loc = self._B_full[:, :k]
        _, b_need = self._side_tables(p.col, "B")
        # A rows stay where they are: reference = owner rank << 25 | row inside the owner's block
        if max(int(p.row.peer_owned.max(initial=0)), p.row.n_owned) >= 1 << 25:
            raise ValueError("more than 2^25 owned rows on one rank")
        row_ranks = np.asarray(_peer_ranks(p, "row"), dtype=np.int64)
        if self.stage_a:
            refs = None    # every A row the kernel touches is in my own block: no reference table
        else:
            refs = np.concatenate([(self.rank << 25) | np.arange(p.row.n_owned, dtype=np.int64),
                                   (row_ranks[p.row.recv_peer] << 25) | p.row.recv_src_idx.astype(np.int64)])
        _, a_need = self._side_tables(p.row, "A")
        self.a_src = self._dev_i64(a_need if a_need.size else [0])
        self.a_refs = None if refs is None else self._dev_i32(refs if refs.size else [0])
        self.a_bases = self._dev_i64([h.addr("A", r) for r in range(h.world)])
        self.b_src = self._dev_i64(b_need if b_need.size else [0])
        self.zwidth = p.nnz // Z + (1 if p.nnz % Z else 0)
        fiber = _peer_ranks(p, "fiber")
        self.zbuf_ptrs = self._dev_i64([h.addr("zbuf", r) for r in fiber])
        self.out_len = p.nnz if Z == 1 else p.owned_nnz_slice()[1]
        self.out = torch.zeros(max(self.out_len, 1), dtype=self.dtype, device=self.device)
        a = self.args = _SddmmArgs()
        row_r, col_r = _peer_ranks(p, "row"), _peer_ranks(p, "col")
        read_from = [row_r[q] for q in range(p.row.npeers) if p.row.recv_counts[q] > 0] + \
                    [col_r[q] for q in range(p.col.npeers) if p.col.recv_counts[q] > 0]
        readers = [row_r[q] for q in range(p.row.npeers) if p.row.send_counts[q] > 0] + \
                  [col_r[q] for q in range(p.col.npeers) if p.col.send_counts[q] > 0]
        others = [r for r in fiber if r != self.rank] if Z > 1 else []
        self._fill_comm(a.comm, read_from, readers, others, others)
        a.nnz = p.nnz
        # with rows to pull, the nonzeros are re-ordered by the pull wave that completes them (`_plan_waves`):
        # what needs no pulled row is computed while the pulls are in flight
        n_recv_a = p.row.n_recv if self.stage_a else 0
        a.n_recv_a, a.a_src = n_recv_a, self.a_src.data_ptr()
        a.A_stage = self._A_full.data_ptr() + p.row.n_owned * self.row_bytes
        a.pull_order, a.n_waves, a.tiles_per_wave, a.wave_nnz = None, 0, 0, None
        self._pull_config(a.pull)
        self.value_order = None   # None: results are stored in the plan's CSR order
        if overlap and (p.col.n_recv + n_recv_a) > 0 and p.nnz > 0:
            order, wave_nnz = self._plan_waves(p, n_recv_a)
            # the kernel walks the nonzeros class by class and stores its values in that order: `value_order`
            # is the storage order of this op's result (position in the plan's CSR order of every value)
            self.value_order = order
            order_dev = torch.from_numpy(order).to(self.device)    # the gathers run on the device
            self._perm = (op.rowidx.index_select(0, order_dev), op.colidx.index_select(0, order_dev),
                          op.vals.index_select(0, order_dev))
            del order_dev
            a.rowidx, a.colidx, a.sval = (t.data_ptr() for t in self._perm)
            a.orig = None
            a.nnz_free = int(wave_nnz[0])
            a.work_per_pull = 1
            a.wave_nnz = self._wave_nnz.data_ptr()
            a.pull_order = self._pull_order.data_ptr()
        else:
            a.rowidx, a.colidx, a.sval = op.rowidx.data_ptr(), op.colidx.data_ptr(), op.vals.data_ptr()
            a.orig, a.nnz_free, a.work_per_pull = None, 0, 1 << 30
        a.a_refs = None if self.a_refs is None else self.a_refs.data_ptr()
        a.a_bases, a.world = self.a_bases.data_ptr(), h.world
        a.B_loc, a.ldb = self._B_full.data_ptr(), kp
        a.n_owned_b, a.n_recv_b = p.col.n_owned, p.col.n_recv
        a.b_src = self.b_src.data_ptr()
        a.nvec = self.nvec
        a.Z, a.my_z = Z, z
        a.zbase, a.zrem = p.nnz // Z, p.nnz % Z
        a.zwidth = self.zwidth
        a.zbuf = self.zbuf_ptrs.data_ptr()
        a.out = self.out.data_ptr()
        self._mc = None
        if Z > 1 and self.zreduce == "multimem":
            if self.dtype != torch.float32:
                raise ValueError("zreduce='multimem' is built for fp32")
            self.part, a.mc_part, a.part_stride = self._multicast_part(op, p.nnz)
        else:
            self.part = torch.zeros(p.nnz if Z > 1 else 1, dtype=self.dtype, device=self.device)
            a.mc_part, a.part_stride = None, 0
        a.part = self.part.data_ptr()
        # Push mode of the partial values (Z > 1).  1: remote stores as the values are computed -- a lane group
        # stores (k_loc/8) consecutive values at a time, which only pays for >= 32 bytes; 0: staged in `part`,
        # pushed in bulk after all of them are there; 2: staged, every warp pushes the contiguous range of its
        # ticket right after computing it (only without the reordering for pull/compute overlap).
        if direct_push is None and "SP3_FUSED_PUSH" in os.environ:
            direct_push = int(os.environ["SP3_FUSED_PUSH"])
        if direct_push is None:
            direct_push = 2 if not a.orig else (1 if self.row_bytes >= 256 else 0)
        direct_push = int(direct_push)
        if direct_push == 2 and a.orig:
            direct_push = 0
        if Z > 1 and self.zreduce == "multimem":
            direct_push = 3   # nothing is pushed: the slice owners reduce through the multicast address
        a.direct_push = self.push_mode = direct_push

    def _plan_waves(self, p, n_recv_a: int, target_waves: int | None = None):
        """Order of the pull tiles, their grouping into waves, and the order of the nonzeros by the wave that
        completes them.  Returns (order, wave_nnz): `order` lists the nonzeros class by class (class 0: both
        dense rows owned; class c: the later of its two rows arrives with wave c - 1), each class in the
        plan's row-sorted order; wave_nnz[c] = nonzeros of classes 0..c.

        Tiles of A rows and tiles of B rows are interleaved in proportion, so that both operands arrive at the
        same relative pace and a nonzero whose two rows come early in their receive lists is ready early."""
        if target_waves is None:
            target_waves = int(os.environ.get("SP3_FUSED_WAVES", "4"))
        target_waves = max(1, min(MAX_WAVES, target_waves))
        n_a, n_b = -(-n_recv_a // self.tile_rows), -(-p.col.n_recv // self.tile_rows)
        n_pull = n_a + n_b
        pos_a, pos_b = np.empty(n_a, np.int64), np.empty(n_b, np.int64)   # place of every tile in its side's sequence
        pos_a[_tiles_by_peer_distance(p.row, n_a, self.tile_rows)] = np.arange(n_a)
        pos_b[_tiles_by_peer_distance(p.col, n_b, self.tile_rows)] = np.arange(n_b)
        key = np.concatenate([(pos_a + 0.5) / max(n_a, 1), (pos_b + 0.5) / max(n_b, 1)])
        code = np.concatenate([np.arange(n_a, dtype=np.int64) | (1 << 30), np.arange(n_b, dtype=np.int64)])
        seq = np.argsort(key, kind="stable")
        pull_order = code[seq]
        tpw = -(-n_pull // target_waves)
        n_waves = -(-n_pull // tpw)
        ticket_of = np.empty(n_pull, np.int64)     # ticket number of tile i (A tiles first, then B tiles)
        ticket_of[seq] = np.arange(n_pull)
        wave_a, wave_b = ticket_of[:n_a] // tpw, ticket_of[n_a:] // tpw
        cls = np.zeros(p.nnz, np.int8)
        rem_b = p.colidx >= p.col.n_owned
        cls[rem_b] = wave_b[(p.colidx[rem_b] - p.col.n_owned) // self.tile_rows] + 1
        if n_recv_a:
            rem_a = p.rowidx >= p.row.n_owned
            ca = np.zeros(p.nnz, np.int8)
            ca[rem_a] = wave_a[(p.rowidx[rem_a] - p.row.n_owned) // self.tile_rows] + 1
            np.maximum(cls, ca, out=cls)
        order = np.argsort(cls, kind="stable")
        wave_nnz = np.cumsum(np.bincount(cls, minlength=n_waves + 1)).astype(np.int64)
        self._pull_order = self._dev_i32(pull_order)
        self._wave_nnz = self._dev_i64(wave_nnz)
        self.args.n_waves, self.args.tiles_per_wave = int(n_waves), int(tpw)
        self.wave_nnz = wave_nnz
        return order, wave_nnz

    def _multicast_part(self, op, nnz: int):
        """Partial-value buffer [2][nnz rounded up to 4] in torch symmetric memory, bound to a multicast object
        over the Z fiber (NVLS).  Returns (local tensor, multicast address, values per half)."""
        group = getattr(op, "_fiber_group", None)
        if group is None:
            raise ValueError("zreduce='multimem' needs the fiber process group (real ranks, not emulation)")
        import torch.distributed._symmetric_memory as symm_mem
        stride = (nnz + 3) // 4 * 4
        t = symm_mem.empty(2 * max(stride, 4), dtype=torch.float32, device=self.device)
        hdl = symm_mem.rendezvous(t, group=group)
        mc = int(hdl.multicast_ptr)
        if mc == 0:
            raise ValueError("zreduce='multimem': this system gives no multicast (NVLS) address")
        t.zero_()
        self._mc = hdl
        return t, mc, stride

    def release(self):
        """Drops the multicast binding (collective over the fiber when zreduce='multimem'): call it on every
        rank, with no kernel in flight, before a rank exits."""
        if self._mc is not None:
            torch.cuda.synchronize(self.device)
            self._mc, self.part = None, None

    def launch(self, phases=PH_ALL, new_epoch=True):
        if new_epoch:
            self.epoch += 1
        self._launch(self._fn("sddmm"), phases)

    def run(self):
        self.launch()
        return self.out[:self.out_len]


class FusedSpMM(_FusedBase):
    """reduce="slots" (default): partial rows of rows owned elsewhere go to a slot at the owner, which adds
    them in ascending source order (bitwise reproducible).  reduce="atomic": the result lives in the symmetric
    heap (`Y_heap`) and partial rows are added into the owners' rows with atomics -- no slot memory, no second
    pass, results depend on the order of the additions."""

    @staticmethod
    def region_sizes(plan, k_loc: int, reduce: str | None = None, dtype=torch.float32) -> dict:
        rb = _pad4(k_loc, dtype) * _esize(dtype)
        if reduce is None:
            reduce = os.environ.get("SP3_FUSED_SPMM_REDUCE", "slots")
        if reduce == "atomic":
            return {"pad": F_KINDS * MAX_RANKS * 4, "X": plan.col.n_local * rb, "slots": 0,
                    "Y": _align(max(1, plan.row.n_owned) * rb)}
        return {"pad": F_KINDS * MAX_RANKS * 4, "X": plan.col.n_local * rb,
                "slots": 2 * _align(plan.row.n_send * rb)}

    def region_sizes_for(self, plan, k_loc):
        return self.region_sizes(plan, k_loc, self.reduce, dtype=self.dtype)

    def __init__(self, op, heap: SymmHeap | None = None, fabric=None, timeout_s: float = 30.0,
                 reduce: str | None = None, red_v4: bool | None = None, bulk_pull: bool | None = None,
                 overlap: bool = True):
        self.bulk_pull = _bulk_default(bulk_pull)
        if reduce is None:
            reduce = os.environ.get("SP3_FUSED_SPMM_REDUCE", "slots")
        if reduce not in ("slots", "atomic"):
            raise ValueError(f"reduce must be 'slots' or 'atomic', got {reduce!r}")
        self.reduce, self.atomic = reduce, reduce == "atomic"
        if red_v4 is None:
            red_v4 = os.environ.get("SP3_FUSED_RED_V4", "1") == "1"
        super().__init__(op, heap, fabric, timeout_s)
        p, h, k, rb = self.plan, self.heap, self.k_loc, self.row_bytes
        rp = p.row
        if self.atomic and "Y" not in h.sizes:
            raise ValueError("the heap was sized for reduce='slots'")
        kp = self.kpad
        self._X_full = h.view("X", self.dtype, (p.col.n_local, kp))   # padded storage, see _pad4
        self.X_loc = self._X_full[:, :k]
        # no local Y block: owned rows are written straight into the result, the others into their owners' slots
        self.Y_loc = None
        _, x_need = self._side_tables(p.col, "X")
        self.x_src = self._dev_i64(x_need if x_need.size else [0])
        half = h.sizes["slots"] // 2
        assert half % 16 == 0
        row_r, col_r = _peer_ranks(p, "row"), _peer_ranks(p, "col")
        # destination of every partial row I do not own: its slot in the owner's heap
        roff = rp.recv_offsets()
        i_in_seg = np.arange(rp.n_recv, dtype=np.int64) - roff[rp.recv_peer]
        slot_row = rp.push_offset[rp.recv_peer] + i_in_seg
        if self.atomic:
            _, y_dst = self._side_tables(rp, "Y")   # address of every row I do not own inside its owner's Y
            self.Y_heap = h.view("Y", self.dtype, (rp.n_owned, kp))[:, :k]
        else:
            base = np.asarray(h.peer_base, dtype=np.int64) + h.offsets["slots"]
            y_dst = base[np.asarray(row_r, dtype=np.int64)[rp.recv_peer]] + slot_row * rb
            self.Y_heap = None
        self.y_dst = self._dev_i64(y_dst if y_dst.size else [0])
        # contributions to my owned rows: slot rows grouped by owned row, ascending source
        order = np.argsort(rp.send_idx, kind="stable")
        counts = np.bincount(rp.send_idx, minlength=rp.n_owned)
        crows = np.flatnonzero(counts)
        cptr = np.zeros(crows.size + 1, np.int64)
        np.cumsum(counts[crows], out=cptr[1:])
        self.cptr = self._dev_i64(cptr)
        self.crows = self._dev_i32(crows if crows.size else [0])
        self.cslot = self._dev_i32(order if order.size else [0])
        a = self.args = _SpmmArgs()
        self._pull_config(a.pull)
        # Work items.  With rows to pull, the items are ordered by the pull wave that completes them and the
        # nonzeros of long rows are sorted so that their owned columns come first: the kernel then works on
        # what is there while the X rows arrive.  The re-ordered column indices and values are private copies
        # (`_val_perm` maps them to the op's CSR arrays; `refresh_values` follows a change of the values).
        self._val_perm, a.n_waves, a.tiles_per_wave, a.wave_items, a.pull_order = None, 0, 0, None, None
        if os.environ.get("SP3_FUSED_SPMM_WAVES") == "0":   # tuning: no overlap, compute after the last pull
            overlap = False
        if overlap and p.col.n_recv > 0 and p.nnz > 0:
            target = max(1, min(MAX_WAVES, int(os.environ.get("SP3_FUSED_SPMM_WAVES", "4"))))
            n_pull = -(-p.col.n_recv // self.tile_rows)
            tpw = -(-n_pull // target)
            n_waves = -(-n_pull // tpw)
            pull_order = _tiles_by_peer_distance(p.col, n_pull, self.tile_rows)
            ticket_of = np.empty(n_pull, np.int64)
            ticket_of[pull_order] = np.arange(n_pull)
            cls = np.zeros(p.nnz, np.int8)
            rem = p.colidx >= p.col.n_owned
            cls[rem] = ticket_of[(p.colidx[rem] - p.col.n_owned) // self.tile_rows] // tpw + 1
            perm, items, first, npieces, class_items = cuda_ops.build_spmm_wave_items(p.rowptr, cls, n_waves + 1)
            self.sched = cuda_ops.SpmmSchedule(op.rowptr, arrays=(items, first, npieces))
            self._val_perm = torch.from_numpy(perm).to(self.device)
            self._colidx = op.colidx.index_select(0, self._val_perm)
            self._vals = op.vals[self._val_perm]
            self._wave_items = self._dev_i32(class_items)
            a.n_waves, a.tiles_per_wave, a.wave_items = int(n_waves), int(tpw), self._wave_items.data_ptr()
            self._pull_order = self._dev_i32(pull_order)
            a.pull_order = self._pull_order.data_ptr()
        else:
            self.sched = cuda_ops.SpmmSchedule(op.rowptr)
            self._colidx, self._vals = op.colidx, op.vals
        carry, ldc = self.sched.carry_for(kp, self.dtype, self.device)
        self.slots = h.view("slots", self.dtype, (h.sizes["slots"] // self.es,))
        flag = np.zeros(max(1, rp.n_owned), np.uint8)
        flag[crows] = 1
        self.crow_flag = torch.from_numpy(flag).to(self.device)
        read_from = [col_r[q] for q in range(p.col.npeers) if p.col.recv_counts[q] > 0]
        readers = [col_r[q] for q in range(p.col.npeers) if p.col.send_counts[q] > 0]
        push_to = [row_r[q] for q in range(rp.npeers) if rp.recv_counts[q] > 0]
        contrib = [row_r[q] for q in range(rp.npeers) if rp.send_counts[q] > 0]
        self._fill_comm(a.comm, read_from, readers, push_to, contrib)
        a.nitems, a.items = self.sched.items.shape[0], self.sched.items.data_ptr()
        a.rowptr, a.colidx, a.val = op.rowptr.data_ptr(), self._colidx.data_ptr(), self._vals.data_ptr()
        a.X_loc, a.ldx = self._X_full.data_ptr(), kp
        a.n_owned_x, a.n_recv_x = p.col.n_owned, p.col.n_recv
        a.x_src = self.x_src.data_ptr()
        a.nvec = self.nvec
        a.lg.first_piece, a.lg.npieces = self.sched.first.data_ptr(), self.sched.npieces.data_ptr()
        a.lg.counters = self.sched.counters.data_ptr()
        a.lg.carry = carry.data_ptr() if carry is not None else None
        a.lg.ldc = ldc if carry is not None else kp
        a.lg.piece_len = self.sched.piece_len
        a.n_owned_y = rp.n_owned
        a.n_crows, a.crows = int(crows.size), self.crows.data_ptr()
        a.y_dst = self.y_dst.data_ptr()
        a.parity_off_v = half // 16
        a.cptr, a.cslot = self.cptr.data_ptr(), self.cslot.data_ptr()
        a.slots, a.lds = self.slots.data_ptr(), kp
        a.atomic, a.red_v4, a.crow_flag = int(self.atomic), int(bool(red_v4)), self.crow_flag.data_ptr()
        if self.atomic:
            a.parity_off_v = 0

    def refresh_values(self):
        """Call after the values of the sparse matrix (`DistSpMM.vals`) were changed: the kernel reads a copy
        of them in its own order when it overlaps pulls with compute."""
        if self._val_perm is not None:
            torch.index_select(self.op.vals, 0, self._val_perm, out=self._vals)

    def launch(self, Y: torch.Tensor, beta: float, phases=PH_ALL, new_epoch=True):
        if new_epoch:
            self.epoch += 1
        a = self.args
        if self.atomic and Y.data_ptr() != self.Y_heap.data_ptr():
            raise ValueError("reduce='atomic': the result must be this op's Y_heap (peers add into it)")
        ldy = Y.stride(0) if Y.shape[0] > 1 else self.kpad
        if (ldy * self.es) % 16 or ldy < self.kpad or Y.data_ptr() % 16 or Y.dtype != self.dtype:
            raise ValueError(f"the result needs a 16-byte aligned base, rows that are a multiple of 16 bytes apart "
                             f"and a leading dimension of at least {self.kpad} (use DistSpMM.Y_owned)")
        a.Y, a.ldy, a.beta = Y.data_ptr(), ldy, float(beta)
        self._launch(self._fn("spmm"), phases)

    def run(self, Y: torch.Tensor, beta: float = 0.0):
        self.launch(Y, beta)
        return Y


def run_lockstep(fused_ops, launch_args=None):
    """Runs one epoch of every given fused op (all ranks of a LocalFabric mesh,
    on one GPU and one stream) phase by phase: START of every rank, then MAIN
    of every rank, then FINISH of every rank.  No launch waits for a later
    one."""
    launch_args = launch_args or [()] * len(fused_ops)
    for i, phase in enumerate((PH_START, PH_MAIN, PH_FINISH)):
        for f, args in zip(fused_ops, launch_args):
            f.launch(*args, phases=phase, new_epoch=(i == 0))
