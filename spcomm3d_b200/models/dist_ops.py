"""Distributed 3D SDDMM and SpMM.

One object per (plan, k, dtype, variant).  The plan is built once per
(matrix, mesh); an op built from it is run many times, like the reference's
"setup once, iterate" contract (miniapp/bench_both.cpp:172-236,
miniapp/bench_spmm.cpp:166-188).

    C = S o (A B^T)        DistSDDMM   (src/distributed_comp.cpp:141-284, 349-413)
    Y = S X                DistSpMM    (src/distributed_comp.cpp:17-76, 285-348)

Dense operands live in *owner layout*: rank (x, y, z) holds the rows it owns
(`plan.row.owned_gids` for A / Y, `plan.col.owned_gids` for B / X) and the
z-th slice of the k columns.  Variants:

  "sparse"     packed exchange with send and receive staging   (ref "sparse")
  "sparseNRB"  packed exchange, received rows land in place    (ref "sparseNRB")
  "fused"      one sm_100a kernel per op that pulls the needed rows from the
               owners' memory over NVLink, computes, and pushes partial
               results to their owners (zero staging; the role of ref
               "sparseNB"); needs GPUs with peer access
  "fused-atomic"  the fused kernels with the SpMM partial rows added into the
               owners' result rows by atomics (no slot memory, no second pass,
               sums not bitwise reproducible)
  "fused-multimem"  the fused kernels with the SDDMM Z reduction done inside the
               NVSwitch: partial values stay in a multicast-bound buffer and the
               slice owners read them with `multimem.ld_reduce.add` (NVLS)
  "dense"      sparsity-agnostic: all-gather whole slabs, reduce-scatter
               (ref "dense", src/dcomm_setup.cpp)

SDDMM result: after the Z reduction fiber rank z holds the z-th contiguous
slice of the block's values in the op's storage order: the plan's CSR order
for the library variants; the fused variant stores values in the order it
computes them and says which value is where (`value_order`,
`owned_positions()`).  SpMM result: owned rows
of Y; partial rows are summed at the owner in ascending peer order.  (The
reference's sparse SpMM post step sends a stale buffer,
src/distributed_comp.cpp:59; here it is defined by the math.)
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..ops import local
from ..parallel.comm import CombinedExpand, DenseExchange, FiberReduce, PhaseTimer, SparseExchange
from ..parallel.mesh import MeshGroups, split_k
from ..parallel.plan import RankPlan
from ..utils import generate

VARIANTS = ("sparse", "sparseNRB", "fused", "dense")
ALG_NAMES = {"sparse": "sparse", "sparseNRB": "sparseNRB", "fused": "sparseNB", "dense": "dense"}


def _library_path_on_fiber_only_mesh(variant: str, plan, kw: dict) -> bool:
    """Meshes 1 x 1 x Z move no dense row: the SDDMM needs only the reduce-scatter of its partial values along the
    fiber, the SpMM no communication at all.  A library reduce-scatter (NCCL, NVLS-capable) is at least as fast
    there as remote stores plus a local sum (measured: 0.50 against 0.52 ms on 2 GPUs, 1.56 against 2.18 ms on 4),
    and the plain local kernels are 5-10 % faster than the fused kernels with nothing to pull.  So on these meshes
    the variant "fused" runs the library path; pass force_fused=True (or use the emulation's heaps) to run the
    fused kernels anyway."""
    return (variant == "fused" and plan.mesh.X == 1 and plan.mesh.Y == 1 and plan.mesh.Z > 1
            and kw.get("heap") is None and not kw.get("force_fused"))


class _Dist3DOp:
    kernel = "?"

    def __init__(self, plan: RankPlan, groups: MeshGroups | None, k: int, dtype=torch.float32,
                 device="cpu", variant: str = "sparseNRB", emulated: bool = False, check_plan: bool = True):
        if variant not in VARIANTS:
            raise ValueError(f"variant must be one of {VARIANTS}")
        self.plan, self.groups, self.k, self.dtype, self.variant = plan, groups, k, dtype, variant
        self.device = torch.device(device)
        self.mesh = plan.mesh
        self.k_off, self.k_loc = split_k(k, self.mesh.Z, plan.coords[2])
        self.timer = PhaseTimer(self.device)
        self.last_times: dict = {}
        # True: `run` does not raise on a status recorded by a fused kernel; `close` raises it, after all ranks
        # have dropped what binds their memory to each other
        self.defer_status = False
        if groups is None and self.mesh.size != 1 and not emulated:
            raise ValueError("a multi-rank mesh needs MeshGroups")
        if groups is not None and check_plan and not plan.meta.get("consistent"):
            # collective, once per plan: same mesh, matrix and seed on every rank before anything is launched
            from ..parallel import health
            health.check_consistent(plan, groups)
            plan.meta["consistent"] = True
        if variant == "fused" and self.device.type != "cuda":
            raise ValueError("the fused variant runs on GPUs only")
        self.rowptr = torch.from_numpy(plan.rowptr).to(self.device)
        self.vals = torch.from_numpy(plan.vals).to(device=self.device, dtype=dtype)
        rowidx, colidx = plan.rowidx, plan.colidx
        self._row_group = groups.row if groups else None
        self._col_group = groups.col if groups else None
        self._fiber_group = groups.fiber if groups else None
        self._dense_row = self._dense_col = None
        if variant == "dense":
            self._dense_row = DenseExchange(plan.row, self._row_group, self.k_loc, dtype, self.device)
            self._dense_col = DenseExchange(plan.col, self._col_group, self.k_loc, dtype, self.device)
            rowidx = self._dense_row.slab_index()[rowidx].astype(np.int32)
            colidx = self._dense_col.slab_index()[colidx].astype(np.int32)
        self.rowidx = torch.from_numpy(np.ascontiguousarray(rowidx)).to(self.device)
        self.colidx = torch.from_numpy(np.ascontiguousarray(colidx)).to(self.device)
        if self.device.type == "cuda" and os.environ.get("SP3_DEBUG") == "1" and variant != "dense":
            from ..ops import cuda_ops
            cuda_ops.validate_indices(self.rowidx, self.colidx, plan.row.n_local, plan.col.n_local)

    # ---- helpers ---------------------------------------------------------
    def _alloc_local(self, side):
        return torch.zeros(side.n_local, self.k_loc, dtype=self.dtype, device=self.device)

    def _exchange(self, side, group):
        mode = "buffered" if self.variant == "sparse" else "nrb"
        return SparseExchange(side, group, self.k_loc, self.dtype, self.device, mode, self.timer)

    def fill_owned(self, target: torch.Tensor, gids, *, kind=generate.FILL_NORMAL, const=0.0, seed=0, stream=0):
        """Writes rows `gids`, my k slice, of the virtual global operand
        defined by (seed, stream) into `target`."""
        npdt = np.float32 if self.dtype == torch.float32 else np.float64
        host = generate.fill_rows(gids, self.k, self.k_off, self.k_loc, kind=kind, const=const, seed=seed,
                                  stream=stream, dtype=npdt)
        target.copy_(torch.from_numpy(host))
        return target

    def poison_unowned(self):
        """NaN-fills every non-owned row so a missed transfer shows up."""
        for buf, side in self._local_buffers():
            buf[side.n_owned:].fill_(float("nan"))

    def _finish(self):
        if not self.timer.enabled:
            return None
        if self.variant == "fused" and not self.defer_status:
            self._fused.check()
        self.last_times = self.timer.collect()
        t = self.last_times
        t["total"] = t.get("comm1", 0.0) + t.get("comp", 0.0) + t.get("comm2", 0.0)
        return t

    def run_async(self, *a, **kw):
        """`run` without phase timers: no host synchronisation, for callers
        that time a whole loop themselves."""
        self.timer.enabled = False
        try:
            return self.run(*a, **kw)
        finally:
            self.timer.enabled = True

    def close(self):
        """Collective shutdown: every rank calls it, with none of its kernels in flight.  Synchronises, meets
        the other ranks, drops what binds this rank's memory to its peers (the NVLink multicast binding of the
        in-switch Z reduction), and meets them again, so that no rank leaves while its memory is still bound.
        A status recorded by a fused kernel is raised only after the release."""
        f = getattr(self, "_fused", None)
        if f is None:
            return
        import torch.distributed as dist
        err = None
        try:
            f.check()
        except Exception as e:  # report after the collective release
            err = e
        multi = self.groups is not None and dist.is_initialized()
        if multi:
            dist.barrier()
        if hasattr(f, "release"):
            f.release()
        if multi:
            dist.barrier()
        if err is not None:
            raise err

    def alg_name(self, phase: str) -> str:
        name = getattr(self, "requested_variant", self.variant)
        name = "fused" if name.startswith("fused") else name
        return f"{ALG_NAMES[name]} {self.kernel} {phase}"


class DistSDDMM(_Dist3DOp):
    kernel = "sddmm"

    def __init__(self, plan, groups, k, dtype=torch.float32, device="cpu", variant="sparseNRB", **kw):
        if variant == "fused-atomic":  # only SpMM has an atomic mode
            variant = "fused"
        requested = variant
        if variant == "fused-multimem":  # Z reduction of the partial values inside the NVSwitch
            variant, kw = "fused", {**kw, "zreduce": "multimem", "force_fused": True}
        if _library_path_on_fiber_only_mesh(variant, plan, kw):
            variant = "sparseNRB"
        super().__init__(plan, groups, k, dtype, device, variant, emulated=kw.get("heap") is not None,
                         check_plan=kw.get("check_plan", True))
        self.requested_variant = requested
        p = plan
        if variant == "fused":
            from ..ops.fused import FusedSDDMM
            self._fused = FusedSDDMM(self, **{k_: v for k_, v in kw.items() if k_ in (
                "heap", "fabric", "timeout_s", "overlap", "direct_push", "stage_a", "zreduce", "bulk_pull")})
            self.A_loc, self.B_loc = self._fused.A_loc, self._fused.B_loc
        else:
            self.A_loc, self.B_loc = self._alloc_local(p.row), self._alloc_local(p.col)
        self.A_owned, self.B_owned = self.A_loc[:p.row.n_owned], self.B_loc[:p.col.n_owned]
        self.partial = torch.zeros(p.nnz, dtype=dtype, device=self.device)
        self.exAB = None
        if variant in ("sparse", "sparseNRB"):
            self.exA = self._exchange(p.row, self._row_group)
            self.exB = self._exchange(p.col, self._col_group)
            # "sparse": A and B rows in one exchange over the plane, as the reference's combined handle does
            # (src/comm_setup.cpp:434-577); the batched point-to-point transport keeps the two line exchanges
            if (variant == "sparse" and groups is not None and self.mesh.xy_size > 1
                    and os.environ.get("SP3_TRANSPORT", "alltoall") == "alltoall"):
                self.exAB = CombinedExpand(p.row, p.col, groups.plane, self.mesh, p.coords, self.k_loc, dtype,
                                           self.device, self.timer)
        if variant != "fused":
            self.fiber = FiberReduce(p.nnz, self.mesh.Z, p.coords[2], self._fiber_group, dtype, self.device)
        # opt-in: dense (128-row x 64-column) panels on the tensor cores (TF32), the rest on the gather kernel
        self._panels = None
        if kw.get("panels") and variant in ("sparse", "sparseNRB") and self.device.type == "cuda":
            from ..ops.panel import PanelSDDMM
            self._panels = PanelSDDMM(p.rowidx, p.colidx, p.vals, p.row.n_local, p.col.n_local, self.device,
                                      **{k_: v for k_, v in kw.items() if k_ in ("min_col_nnz", "min_panel_nnz")})
        self.owned_off, self.owned_len = p.owned_nnz_slice()

    def _local_buffers(self):
        return [(self.A_loc, self.plan.row), (self.B_loc, self.plan.col)]

    def run(self) -> torch.Tensor:
        """One distributed SDDMM; returns my slice of C's values."""
        t = self.timer
        if self.variant == "fused":
            with t.span("comp"):
                c = self._fused.run()
        elif self.variant == "dense":
            with t.span("comm1"):
                A = self._dense_row.all_gather(self.A_owned)
                B = self._dense_col.all_gather(self.B_owned)
            with t.span("comp"):
                local.sddmm(self.rowidx, self.colidx, self.vals, A, B, out=self.partial)
            with t.span("comm2"):
                c = self.fiber(self.partial)
        else:
            with t.span("comm1"):
                if self.exAB is not None:
                    self.exAB.expand(self.A_loc, self.B_loc)
                else:
                    self.exA.expand(self.A_loc)
                    self.exB.expand(self.B_loc)
            with t.span("comp"):
                if self._panels is not None:
                    self._panels.run(self.A_loc, self.B_loc, self.partial)
                else:
                    local.sddmm(self.rowidx, self.colidx, self.vals, self.A_loc, self.B_loc, out=self.partial)
            with t.span("comm2"):
                c = self.fiber(self.partial)
        if self.mesh.Z == 1:
            c = c[self.owned_off:self.owned_off + self.owned_len]
        self._finish()
        return c

    @property
    def value_order(self):
        """Storage order of the result values: None when they are in the plan's CSR order (library variants),
        else an int64 array giving, for every stored value of the block, its position in the plan's CSR order
        (the fused kernel stores its values in the order in which it computes them: nonzeros whose dense rows
        are owned first, then the others by the pull wave that completes them)."""
        f = getattr(self, "_fused", None)
        return None if f is None else f.value_order

    def owned_positions(self) -> np.ndarray:
        """Positions, in the plan's CSR order, of the values `run` returns on this rank (after the Z reduction
        fiber rank z holds the z-th contiguous slice of the block's values in storage order)."""
        pos = np.arange(self.owned_off, self.owned_off + self.owned_len, dtype=np.int64)
        order = self.value_order
        return pos if order is None else np.asarray(order[pos], dtype=np.int64)

    def comm_stats(self):
        """{'PRE': ((send_msgs, send_vol), (recv_msgs, recv_vol)), 'POST': ...}
        in the reference's units (elements)."""
        p, k = self.plan, self.k_loc
        if self.variant == "dense":
            (sa, ra), (sb, rb) = self._dense_row.stats_gather(), self._dense_col.stats_gather()
            pre = ((1, sa[1] + sb[1]), (ra[0] + rb[0], ra[1] + rb[1]))
        else:
            s, r, sm, rm = p.expand_rows()
            pre = ((sm, s * k), (rm, r * k))
        from ..parallel.mesh import split_nnz
        post = ((1, p.nnz), (1, split_nnz(p.nnz, self.mesh.Z, p.coords[2])[1]))
        return {"PRE": pre, "POST": post}

    def flops(self) -> float:
        return 2.0 * self.plan.gnnz * self.k


class DistSpMM(_Dist3DOp):
    kernel = "spmm"

    def __init__(self, plan, groups, k, dtype=torch.float32, device="cpu", variant="sparseNRB", **kw):
        if variant == "fused-atomic":  # the fused kernel with partial rows added into the owners' rows by atomics
            variant, kw = "fused", {**kw, "reduce": "atomic"}
        requested = variant
        if variant == "fused-multimem":  # only SDDMM has a Z reduction
            variant = "fused"
        if _library_path_on_fiber_only_mesh(variant, plan, kw):
            variant = "sparseNRB"
        super().__init__(plan, groups, k, dtype, device, variant, emulated=kw.get("heap") is not None,
                         check_plan=kw.get("check_plan", True))
        self.requested_variant = requested
        p = plan
        if variant == "fused":
            from ..ops.fused import FusedSpMM
            self._fused = FusedSpMM(self, **{k_: v for k_, v in kw.items()
                                             if k_ in ("heap", "fabric", "timeout_s", "reduce", "red_v4", "bulk_pull",
                                                       "overlap")})
            self.X_loc, self.Y_loc = self._fused.X_loc, self._fused.Y_loc
        else:
            self.X_loc, self.Y_loc = self._alloc_local(p.col), self._alloc_local(p.row)
        self.X_owned = self.X_loc[:p.col.n_owned]
        # sparse variants: the result is the owned head of the local Y block (no copy); fused and dense write
        # into a buffer of their own
        if variant in ("sparse", "sparseNRB"):
            self.Y_owned = self.Y_loc[:p.row.n_owned]
        elif variant == "fused" and self._fused.atomic:
            self.Y_owned = self._fused.Y_heap   # peers add their partial rows into it
        elif variant == "fused":
            # same padded leading dimension as the kernel's other dense blocks (any k / Z)
            self.Y_owned = torch.zeros(p.row.n_owned, self._fused.kpad, dtype=dtype,
                                       device=self.device)[:, :self.k_loc]
        else:
            self.Y_owned = torch.zeros(p.row.n_owned, self.k_loc, dtype=dtype, device=self.device)
        self.sched = None
        if variant in ("sparse", "sparseNRB"):
            self.exX = self._exchange(p.col, self._col_group)
            self.exY = self._exchange(p.row, self._row_group)
        if variant == "dense":
            self._Yslab = torch.zeros(p.row.npeers * self._dense_row.max_owned, self.k_loc, dtype=dtype,
                                      device=self.device)
            # CSR over slab rows for the local kernel
            order = np.argsort(self.rowidx.cpu().numpy(), kind="stable")
            ri = self.rowidx.cpu().numpy()[order]
            self._d_rowidx = torch.from_numpy(ri).to(self.device)
            self._d_colidx = self.colidx[torch.from_numpy(order).to(self.device)]
            self._d_vals = self.vals[torch.from_numpy(order).to(self.device)]
            rp = np.zeros(self._Yslab.shape[0] + 1, np.int64)
            np.cumsum(np.bincount(ri, minlength=self._Yslab.shape[0]), out=rp[1:])
            self._d_rowptr = torch.from_numpy(rp).to(self.device)
            self._d_sched = None
        if self.device.type == "cuda" and variant != "fused":
            from ..ops import cuda_ops
            if variant == "dense":
                self._d_sched = cuda_ops.SpmmSchedule(self._d_rowptr)
            else:
                self.sched = cuda_ops.SpmmSchedule(self.rowptr)
        # opt-in: dense (128-row x 64-column) panels of S as TF32 products on the tensor cores
        self._panels = None
        if (kw.get("panels") and variant in ("sparse", "sparseNRB") and self.device.type == "cuda"
                and dtype == torch.float32 and self.k_loc % 32 == 0 and self.k_loc <= 256):
            from ..ops.panel import PanelSpMM
            self._panels = PanelSpMM(p.rowidx, p.colidx, p.vals, p.row.n_local, p.col.n_local, self.device,
                                     **{k_: v for k_, v in kw.items() if k_ in ("min_col_nnz", "min_panel_nnz")})

    def _local_buffers(self):
        return [(self.X_loc, self.plan.col)]

    def values_changed(self):
        """Tell the op that `vals` (the values of S, CSR order) was written to: the fused kernel keeps a
        re-ordered copy.  The library variants read `vals` directly."""
        f = getattr(self, "_fused", None)
        if f is not None:
            f.refresh_values()

    def run(self, beta: float = 0.0) -> torch.Tensor:
        """One distributed SpMM: Y_owned = beta*Y_owned + (S X)[owned rows]."""
        t, p = self.timer, self.plan
        if self.variant == "fused":
            with t.span("comp"):
                self._fused.run(self.Y_owned, beta)
        elif self.variant == "dense":
            with t.span("comm1"):
                X = self._dense_col.all_gather(self.X_owned)
            with t.span("comp"):
                local.spmm(self._d_rowptr, self._d_rowidx, self._d_colidx, self._d_vals, X, self._Yslab, 0.0,
                           self._d_sched)
            with t.span("comm2"):
                if beta == 0.0:
                    self._dense_row.reduce_scatter(self._Yslab, self.Y_owned)
                else:
                    prev = self.Y_owned * beta
                    self._dense_row.reduce_scatter(self._Yslab, self.Y_owned)
                    self.Y_owned += prev
        else:
            prev = self.Y_owned * beta if beta != 0.0 else None
            with t.span("comm1"):
                self.exX.expand(self.X_loc)
            with t.span("comp"):
                if self._panels is not None:
                    self._panels.run(self.X_loc, self.Y_loc, 0.0)
                else:
                    local.spmm(self.rowptr, self.rowidx, self.colidx, self.vals, self.X_loc, self.Y_loc, 0.0,
                               self.sched)
            with t.span("comm2"):
                self.exY.reduce(self.Y_loc)  # adds the peers' partial rows into the owned head = Y_owned
                if prev is not None:
                    self.Y_owned.add_(prev)
        self._finish()
        return self.Y_owned

    def comm_stats(self):
        p, k = self.plan, self.k_loc
        if self.variant == "dense":
            pre = self._dense_col.stats_gather()
            mo = self._dense_row.max_owned
            allv = int(p.row.peer_owned.sum()) * k
            post = ((1, allv), (1, int(p.row.peer_owned[p.row.me]) * k)) if p.row.npeers > 1 else ((0, 0), (0, 0))
        else:
            s, r, sm, rm = p.expand_rows(("col",))
            pre = ((sm, s * k), (rm, r * k))
            # reduce = expand of the row side with roles swapped (src/comm_setup.cpp:778-784)
            s, r, sm, rm = p.expand_rows(("row",))
            post = ((rm, r * k), (sm, s * k))
        return {"PRE": pre, "POST": post}

    def flops(self) -> float:
        return 2.0 * self.plan.gnnz * self.k
