"""Library-collective communication engines (the unfused path).

`SparseExchange` is the sparsity-aware engine: it moves exactly the dense
rows a `SidePlan` lists, with torch.distributed collectives (NCCL on GPUs,
gloo on CPUs).  It plays the role of the reference's SparseComm<T>
(src/comm.hpp:28-199): `expand` = pack + P2P + unpack (copy_to_sendbuff :90,
issue_Irecvs/Sends/Waitall :105-139, copy_from_recvbuff :166), `reduce` = the
role-swapped handle of SpMM's post step with the owner-side sum
(SUM_from_recvbuff :178-189, src/comm_setup.cpp:778-784).  Transport: one
`all_to_all_single` with per-peer split sizes, or batched isend/irecv to the
actual neighbours only (`transport="p2p"`).

Staging modes (the reference's three SDDMM instances,
src/distributed_comp.cpp:141-284):
  "buffered" pack -> exchange -> receive staging -> unpack
  "nrb"      pack -> exchange straight into the local block (the needed rows
             of one peer are contiguous there), no receive staging
The zero-staging instance ("NB", MPI derived datatypes) has no library form
here: its counterpart is the fused kernel that pulls rows from the owner's
memory.

`DenseExchange` is the sparsity-agnostic engine (src/denseComm.hpp:12-50):
all-gather of whole owned slabs along a mesh line and a reduce-scatter along
another.

These engines are the measured baseline of the framework, not its product.
"""
from __future__ import annotations

import os

import time

import numpy as np
import torch
import torch.distributed as dist

from ..ops import local
from .plan import SidePlan


class PhaseTimer:
    """Accumulates milliseconds per named phase; CUDA events on GPU streams,
    perf_counter on the host.  Phases of the reference: comm1 (pre), comp,
    comm2 (post), commcpy (pack/unpack), total (src/basic.hpp:20-22)."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.ms: dict[str, float] = {}
        self._pending = []
        self.enabled = True

    class _Span:
        def __init__(self, timer, name):
            self.t, self.name = timer, name

        def __enter__(self):
            if self.t.cuda:
                torch.cuda.nvtx.range_push(f"sp3:{self.name}")
                self.a = torch.cuda.Event(enable_timing=True)
                self.b = torch.cuda.Event(enable_timing=True)
                self.a.record()
            else:
                self.t0 = time.perf_counter()
            return self

        def __exit__(self, *exc):
            if self.t.cuda:
                self.b.record()
                torch.cuda.nvtx.range_pop()
                self.t._pending.append((self.name, self.a, self.b))
            else:
                self.t.ms[self.name] = self.t.ms.get(self.name, 0.0) + (time.perf_counter() - self.t0) * 1e3
            return False

    def span(self, name):
        return PhaseTimer._Span(self, name) if self.enabled else _NullSpan()

    def collect(self) -> dict:
        """Synchronises (GPU) and returns {phase: ms}, then resets."""
        if self.cuda and self._pending:
            torch.cuda.synchronize()
            for name, a, b in self._pending:
                self.ms[name] = self.ms.get(name, 0.0) + a.elapsed_time(b)
            self._pending = []
        out, self.ms = self.ms, {}
        return out


def _splits(counts, unit=1):
    return [int(c) * unit for c in counts]


class SparseExchange:
    """Sparsity-aware exchange of dense rows along one mesh line with library collectives.

    mode: "buffered" (send and receive staging) or "nrb" (rows land in place).
    transport: "alltoall" -- one `all_to_all_single` with per-peer splits (the role of the reference's
    MPI_Neighbor_alltoallv path, src/comm.hpp:149-156); "p2p" -- one receive and one send per actual neighbour,
    batched (the reference's Irecv / Send / Waitall path, src/comm.hpp:105-139).  Default from SP3_TRANSPORT."""

    def __init__(self, side: SidePlan, group, k_loc: int, dtype, device, mode: str = "nrb", timer=None,
                 transport: str | None = None):
        if mode not in ("buffered", "nrb"):
            raise ValueError("mode must be 'buffered' or 'nrb'")
        transport = transport or os.environ.get("SP3_TRANSPORT", "alltoall")
        if transport not in ("alltoall", "p2p"):
            raise ValueError("transport must be 'alltoall' or 'p2p'")
        self.side, self.group, self.k, self.mode, self.transport = side, group, k_loc, mode, transport
        self.device, self.dtype = torch.device(device), dtype
        self.timer = timer
        self.send_idx = torch.from_numpy(side.send_idx).to(self.device)
        self.send_buf = torch.empty(side.n_send, k_loc, dtype=dtype, device=self.device)
        self.recv_buf = (torch.empty(side.n_recv, k_loc, dtype=dtype, device=self.device)
                         if mode == "buffered" else None)
        self.recv_pos = (torch.arange(side.n_owned, side.n_local, dtype=torch.int64, device=self.device)
                         if mode == "buffered" else None)
        self.send_split = _splits(side.send_counts)
        self.recv_split = _splits(side.recv_counts)
        self.send_off = side.send_offsets()
        self.trivial = side.npeers == 1

    def _span(self, name):
        return self.timer.span(name) if self.timer is not None else _NullSpan()

    def _exchange(self, recv: torch.Tensor, send: torch.Tensor, recv_split, send_split):
        """Rows send[...] to the peers, rows from the peers into recv[...] (both grouped by peer, ascending)."""
        if self.transport == "alltoall":
            dist.all_to_all_single(recv, send, recv_split, send_split, group=self.group)
            return
        ops, ro, so = [], 0, 0
        for p in range(self.side.npeers):
            rc, sc = recv_split[p], send_split[p]
            if p != self.side.me:
                if rc:
                    ops.append(dist.P2POp(dist.irecv, recv[ro:ro + rc], group=self.group, group_peer=p))
                if sc:
                    ops.append(dist.P2POp(dist.isend, send[so:so + sc], group=self.group, group_peer=p))
            ro, so = ro + rc, so + sc
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    # statistics in the reference's units: messages = neighbour counts, volume
    # = elements (rows x k_loc), src/comm_stats.cpp:62-65
    def stats(self, reverse=False):
        s = self.side
        send = (s.out_degree(), s.n_send * self.k)
        recv = (s.in_degree(), s.n_recv * self.k)
        return (recv, send) if reverse else (send, recv)

    def expand(self, buf: torch.Tensor):
        """buf[:n_owned] holds my owned rows; fills buf[n_owned:] with the
        needed rows fetched from their owners."""
        s = self.side
        if self.trivial or (s.n_send == 0 and s.n_recv == 0 and self.group is None):
            return buf
        with self._span("commcpy"):
            local.gather_rows(self.send_idx, buf[:s.n_owned], self.send_buf)
        target = self.recv_buf if self.mode == "buffered" else buf[s.n_owned:]
        self._exchange(target, self.send_buf, self.recv_split, self.send_split)
        if self.mode == "buffered":
            with self._span("commcpy"):
                local.scatter_rows(self.recv_pos, self.recv_buf, buf)
        return buf

    def reduce(self, buf: torch.Tensor):
        """buf holds partial rows for every local row; sends the non-owned
        ones to their owners and adds what peers send into buf[:n_owned]
        (peers in ascending order, so the sum order is fixed)."""
        s = self.side
        if self.trivial:
            return buf
        self._exchange(self.send_buf, buf[s.n_owned:].contiguous(), self.send_split, self.recv_split)
        with self._span("commcpy"):
            owned = buf[:s.n_owned]
            for p in range(s.npeers):
                a, b = int(self.send_off[p]), int(self.send_off[p + 1])
                if b > a:
                    local.scatter_add_rows(self.send_idx[a:b], self.send_buf[a:b], owned)
        return buf


class CombinedExpand:
    """Both operands of an SDDMM in one exchange: the A rows a rank's row-line peers need and the B rows its
    column-line peers need travel in a single all_to_all over the xy plane, through one send and one receive
    staging buffer -- the reference's "sparse" instance (one SparseComm handle for A and B rows,
    src/comm_setup.cpp:434-577, run at src/distributed_comp.cpp:157-165).

    Plane ranks ascend as x * Y + y, so the peers of rank (x, y) come in the order: column-line peers with a
    smaller x, the whole row line, column-line peers with a larger x.  Both staging buffers are laid out that
    way, which makes packing and unpacking three contiguous pieces each."""

    def __init__(self, row: SidePlan, col: SidePlan, plane_group, mesh, coords, k_loc: int, dtype, device, timer=None):
        self.row, self.col, self.group, self.k, self.timer = row, col, plane_group, k_loc, timer
        self.device = torch.device(device)
        X, Y = mesh.X, mesh.Y
        x, y = coords[0], coords[1]
        send = np.zeros(X * Y, np.int64)
        recv = np.zeros(X * Y, np.int64)
        for j in range(Y):
            send[x * Y + j] += row.send_counts[j]
            recv[x * Y + j] += row.recv_counts[j]
        for i in range(X):
            send[i * Y + y] += col.send_counts[i]
            recv[i * Y + y] += col.recv_counts[i]
        self.send_split, self.recv_split = _splits(send), _splits(recv)
        so, ro = col.send_offsets(), col.recv_offsets()
        self.b_send_lo, self.b_recv_lo = int(so[x]), int(ro[x])   # rows for / from column peers with a smaller x
        self.send_idx_a = torch.from_numpy(row.send_idx).to(self.device)
        self.send_idx_b = torch.from_numpy(col.send_idx).to(self.device)
        self.send_buf = torch.empty(row.n_send + col.n_send, k_loc, dtype=dtype, device=self.device)
        self.recv_buf = torch.empty(row.n_recv + col.n_recv, k_loc, dtype=dtype, device=self.device)

    def _span(self, name):
        return self.timer.span(name) if self.timer is not None else _NullSpan()

    def stats(self):
        r, c = self.row, self.col
        return ((r.out_degree() + c.out_degree(), (r.n_send + c.n_send) * self.k),
                (r.in_degree() + c.in_degree(), (r.n_recv + c.n_recv) * self.k))

    def expand(self, A: torch.Tensor, B: torch.Tensor):
        """A[:n_owned], B[:n_owned] hold the owned rows; fills A[n_owned:] and B[n_owned:]."""
        r, c = self.row, self.col
        lo_s, lo_r = self.b_send_lo, self.b_recv_lo
        with self._span("commcpy"):
            if lo_s:
                local.gather_rows(self.send_idx_b[:lo_s], B[:c.n_owned], self.send_buf[:lo_s])
            if r.n_send:
                local.gather_rows(self.send_idx_a, A[:r.n_owned], self.send_buf[lo_s:lo_s + r.n_send])
            if c.n_send > lo_s:
                local.gather_rows(self.send_idx_b[lo_s:], B[:c.n_owned], self.send_buf[lo_s + r.n_send:])
        dist.all_to_all_single(self.recv_buf, self.send_buf, self.recv_split, self.send_split, group=self.group)
        with self._span("commcpy"):
            B[c.n_owned:c.n_owned + lo_r].copy_(self.recv_buf[:lo_r])
            A[r.n_owned:].copy_(self.recv_buf[lo_r:lo_r + r.n_recv])
            B[c.n_owned + lo_r:].copy_(self.recv_buf[lo_r + r.n_recv:])
        return A, B


class _NullSpan:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class DenseExchange:
    """Sparsity-agnostic movement of whole owned blocks along one mesh line.

    The slab is `[npeers, max_owned, k]`: peer p's owned rows sit at
    `slab[p, :peer_owned[p]]`, the tail of each block is padding so that one
    equal-sized all_gather / reduce_scatter serves every peer.  Local index of
    global row g in the slab: `owner(g) * max_owned + pos(g)`, identical on
    all ranks (the reference numbers slab rows inconsistently across ranks,
    src/dcomm_setup.cpp:152-158,185, which made its dense path unverifiable).
    """

    def __init__(self, side: SidePlan, group, k_loc: int, dtype, device):
        self.side, self.group, self.k = side, group, k_loc
        self.max_owned = int(side.peer_owned.max()) if side.npeers else 0
        self.slab = torch.zeros(side.npeers, self.max_owned, k_loc, dtype=dtype, device=device)
        self.pad = torch.zeros(self.max_owned, k_loc, dtype=dtype, device=device)

    def slab_index(self) -> np.ndarray:
        """Slab row of every row of the side's local layout."""
        s = self.side
        own = s.me * self.max_owned + np.arange(s.n_owned, dtype=np.int64)
        need = s.recv_peer.astype(np.int64) * self.max_owned + s.recv_src_idx.astype(np.int64)
        return np.concatenate([own, need])

    def stats_gather(self):
        # bcast model of src/comm_stats.cpp:107-120: own block out once, all other blocks in
        s = self.side
        if s.npeers == 1:
            return (0, 0), (0, 0)
        mine = int(s.peer_owned[s.me]) * self.k
        allv = int(s.peer_owned.sum()) * self.k
        return (1, mine), (s.npeers, allv - mine)

    def all_gather(self, owned: torch.Tensor) -> torch.Tensor:
        s = self.side
        self.pad[:s.n_owned].copy_(owned)
        if s.npeers == 1:
            self.slab[0].copy_(self.pad)
        else:
            dist.all_gather_into_tensor(self.slab.view(-1, self.k), self.pad, group=self.group)
        return self.slab.view(-1, self.k)

    def reduce_scatter(self, slab: torch.Tensor, owned_out: torch.Tensor) -> torch.Tensor:
        """Sums the slab over the line and leaves my owned block in owned_out."""
        s = self.side
        if s.npeers == 1:
            self.pad.copy_(slab.view(s.npeers, self.max_owned, self.k)[0])
        else:
            dist.reduce_scatter_tensor(self.pad, slab.view(-1, self.k), group=self.group)
        owned_out.copy_(self.pad[:s.n_owned])
        return owned_out


class FiberReduce:
    """Sum of partial SDDMM values along the Z fiber; rank z keeps the z-th
    contiguous slice (nnz//Z, +1 for the first nnz%Z).  Library form of the
    reference's MPI_Reduce_scatter on zcomm (src/denseComm.hpp:35-40, counts
    from src/comm_setup.cpp:682-687)."""

    def __init__(self, nnz: int, Z: int, z: int, group, dtype, device):
        from .mesh import split_nnz
        self.nnz, self.Z, self.z, self.group = nnz, Z, z, group
        self.slices = [split_nnz(nnz, Z, i) for i in range(Z)]
        self.width = self.slices[0][1] if Z else 0  # widest slice
        self.even = nnz % Z == 0
        self.out = torch.empty(self.width, dtype=dtype, device=device)
        self.padded = None if self.even else torch.zeros(Z, self.width, dtype=dtype, device=device)
        self._recv = None

    def stats(self):
        # src/comm_stats.cpp:98-105: send all local values, receive own slice, one message
        return (1, self.nnz), (1, self.slices[self.z][1])

    def __call__(self, partial: torch.Tensor) -> torch.Tensor:
        off, ln = self.slices[self.z]
        if self.Z == 1:
            return partial
        if partial.device.type == "cpu":
            # CPU ranks (gloo): exchange the slices and add them in ascending fiber order; gloo's own
            # reduce-scatter costs about twice as much at these sizes
            if self._recv is None:
                self._recv = torch.empty(self.Z * ln, dtype=partial.dtype)
            dist.all_to_all_single(self._recv, partial, [ln] * self.Z, [l for _, l in self.slices], group=self.group)
            torch.sum(self._recv.view(self.Z, ln), dim=0, out=self.out[:ln])
            return self.out[:ln]
        if self.even:
            dist.reduce_scatter_tensor(self.out, partial, group=self.group)
        else:
            for i, (o, l) in enumerate(self.slices):
                self.padded[i, :l].copy_(partial[o:o + l])
            dist.reduce_scatter_tensor(self.out, self.padded.view(-1), group=self.group)
        return self.out[:ln]
