"""Pipelines built from the two distributed kernels.

`SddmmSpmmStep`  one SDDMM followed by one SpMM on the same sparse matrix with
                 its stored values: the unit the benchmarks time (the
                 reference runs the two kernels as separate programs,
                 miniapp/bench_both.cpp and miniapp/bench_spmm.cpp, or back to
                 back in miniapp/main_combined.cpp:165-281).
`GatLayer`       attention-style chain: edge scores C = S o (A B^T), then
                 Y = C X with the scores as the sparse values.  The scores are
                 summed along the Z fiber and then shared by the whole fiber,
                 because every Z layer multiplies the full block with its own
                 slice of X's columns.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from ..parallel.mesh import split_nnz
from .dist_ops import DistSDDMM, DistSpMM

STREAM_A, STREAM_B = 1, 2


class SddmmSpmmStep:
    def __init__(self, plan, groups, k, dtype=torch.float32, device="cuda", variant="sparseNRB", seed=0,
                 **kw):
        self.plan, self.k, self.seed = plan, k, seed
        self.device = torch.device(device)
        self.sddmm = DistSDDMM(plan, groups, k, dtype, device, variant, **kw)
        self.spmm = DistSpMM(plan, groups, k, dtype, device, variant, **kw)
        self.host = None

    def fill_device_operands(self):
        """A, B (and X = B) generated on the device from the seed."""
        sd, sp, p = self.sddmm, self.spmm, self.plan
        if self.device.type == "cuda":
            from ..ops import cuda_ops
            ga = torch.from_numpy(p.row.owned_gids).to(self.device)
            gb = torch.from_numpy(p.col.owned_gids).to(self.device)
            cuda_ops.fill_rows(ga, self.k, sd.k_off, sd.A_owned, seed=self.seed, stream=STREAM_A)
            cuda_ops.fill_rows(gb, self.k, sd.k_off, sd.B_owned, seed=self.seed, stream=STREAM_B)
            sp.X_owned.copy_(sd.B_owned)
        else:
            sd.fill_owned(sd.A_owned, p.row.owned_gids, seed=self.seed, stream=STREAM_A)
            sd.fill_owned(sd.B_owned, p.col.owned_gids, seed=self.seed, stream=STREAM_B)
            sp.X_owned.copy_(sd.B_owned)

    def run_device(self):
        c = self.sddmm.run_async()
        y = self.spmm.run_async()
        return c, y

    # ---- end to end: operands start in pinned host memory -----------------
    def make_host_operands(self):
        sd = self.sddmm
        pin = self.device.type == "cuda"
        self.host = {"A": sd.A_owned.cpu(), "B": sd.B_owned.cpu()}
        if pin:
            self.host = {n: t.pin_memory() for n, t in self.host.items()}
        self._sums = torch.zeros(2, dtype=torch.float64, device=self.device)
        return self.host

    @property
    def h2d_bytes(self):
        h = self.host
        return int(h["A"].numel() * h["A"].element_size() + h["B"].numel() * h["B"].element_size())

    @property
    def d2h_bytes(self):
        return 16

    def run_e2e(self):
        """Copies the step's inputs A and B from pinned host memory (X of the
        SpMM is B: one device-to-device copy), runs SDDMM and SpMM (the SpMM
        overlaps the copy of A) and reads back the checksums of this rank's
        results (two fp64 scalars)."""
        sd, sp, h = self.sddmm, self.spmm, self.host
        if self.device.type == "cuda":
            # B first; while A follows on a copy stream the SpMM (which needs only X = B) already runs
            main = torch.cuda.current_stream(self.device)
            if getattr(self, "_copy_stream", None) is None:
                self._copy_stream = torch.cuda.Stream(self.device)
                self._ev_b, self._ev_a = torch.cuda.Event(), torch.cuda.Event()
            sd.B_owned.copy_(h["B"], non_blocking=True)
            self._ev_b.record(main)
            self._copy_stream.wait_event(self._ev_b)   # also orders this copy of A after the previous step's SDDMM
            with torch.cuda.stream(self._copy_stream):
                sd.A_owned.copy_(h["A"], non_blocking=True)
                self._ev_a.record(self._copy_stream)
            sp.X_owned.copy_(sd.B_owned)
            y = sp.run_async()
            main.wait_event(self._ev_a)
            c = sd.run_async()
        else:
            sd.A_owned.copy_(h["A"], non_blocking=True)
            sd.B_owned.copy_(h["B"], non_blocking=True)
            sp.X_owned.copy_(sd.B_owned)
            c = sd.run_async()
            y = sp.run_async()
        if self.device.type == "cuda":
            from ..ops import cuda_ops
            self._sums[0:1].copy_(cuda_ops.checksum(c))
            self._sums[1:2].copy_(cuda_ops.checksum(y.reshape(-1)))
        else:
            self._sums[0], self._sums[1] = c.double().sum(), y.double().sum()
        return self._sums.cpu().tolist()

    # ---- health, timing breakdown, shutdown --------------------------------
    def check(self):
        """Synchronises and raises `FusedStatusError` if a fused kernel of either op recorded a bad index
        or a wait that ran out since the last check (the asynchronous run path does not look)."""
        for op in (self.sddmm, self.spmm):
            f = getattr(op, "_fused", None)
            if f is not None:
                f.check()

    def phase_ms(self):
        """In-kernel time stamps of the last fused launches: {"sddmm": {"pull", "main", "total"}, "spmm": ...}
        in milliseconds, or None for the library variants."""
        if getattr(self.sddmm, "_fused", None) is None:
            return None
        return {"sddmm": self.sddmm._fused.phase_ms(), "spmm": self.spmm._fused.phase_ms()}

    def local_kernel_ms(self, iters: int = 5):
        """(sddmm_ms, spmm_ms) of the plain local kernels on this rank's block with every dense row already
        in local memory: what the distributed ops would cost if communication were free."""
        from ..ops import local
        sd, sp, p = self.sddmm, self.spmm, self.plan
        dev, dt, kl = self.device, sd.dtype, sd.k_loc
        f = getattr(sd, "_fused", None)
        A = f._A_full[:, :kl] if f is not None else sd.A_loc
        Y = torch.empty(p.row.n_local, kl, dtype=dt, device=dev)
        sched = sp.sched
        if sched is None and dev.type == "cuda":
            sched = sp._fused.sched if getattr(sp, "_fused", None) is not None else None
        out = []
        for fn in (lambda: local.sddmm(sd.rowidx, sd.colidx, sd.vals, A, sd.B_loc, out=sd.partial),
                   lambda: local.spmm(sp.rowptr, sp.rowidx, sp.colidx, sp.vals, sp.X_loc, Y, 0.0, sched)):
            fn()
            if dev.type == "cuda":
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(iters):
                    fn()
                b.record()
                torch.cuda.synchronize(dev)
                out.append(a.elapsed_time(b) / iters)
            else:
                import time
                t0 = time.perf_counter()
                for _ in range(iters):
                    fn()
                out.append((time.perf_counter() - t0) * 1e3 / iters)
        return tuple(out)

    def close(self):
        """Collective shutdown of both ops (see `_Dist3DOp.close`)."""
        self.sddmm.close()
        self.spmm.close()

    def comm_volume_bytes(self):
        """[sddmm expand, sddmm z-reduce, spmm expand, spmm reduce] bytes this
        rank receives per step according to the plan."""
        es = self.sddmm.A_loc.element_size()
        pre, post = (self.sddmm.comm_stats()[p] for p in ("PRE", "POST"))
        z = self.plan.mesh.Z
        zred = (self.plan.nnz - post[1][1]) if z > 1 else 0  # values leaving this rank
        spre, spost = (self.spmm.comm_stats()[p] for p in ("PRE", "POST"))
        return [pre[1][1] * es, zred * es, spre[1][1] * es, spost[1][1] * es]


class GatLayer:
    """Y = (S o (A B^T)) X on the mesh; returns owned rows of Y."""

    def __init__(self, plan, groups, k, dtype=torch.float32, device="cpu", variant="sparseNRB", **kw):
        self.plan, self.groups = plan, groups
        self.sddmm = DistSDDMM(plan, groups, k, dtype, device, variant, **kw)
        # the SpMM values change every run (they are the SDDMM scores): no precomputed value panels here
        self.spmm = DistSpMM(plan, groups, k, dtype, device, variant,
                             **{k_: v for k_, v in kw.items() if k_ != "panels"})
        Z = plan.mesh.Z
        self.slices = [split_nnz(plan.nnz, Z, z) for z in range(Z)]
        self.width = self.slices[0][1]
        dev = torch.device(device)
        self._mine = torch.zeros(self.width, dtype=dtype, device=dev)
        self._all = torch.zeros(Z, self.width, dtype=dtype, device=dev)
        # the SpMM wants its values in CSR order; a fused SDDMM stores them in its own order
        order = self.sddmm.value_order
        self._pos = None if order is None else torch.from_numpy(np.ascontiguousarray(order)).to(dev)

    def run(self):
        c = self.sddmm.run()
        Z = self.plan.mesh.Z
        if Z == 1:
            if self._pos is None:
                self.spmm.vals.copy_(c)
            else:
                self.spmm.vals.index_copy_(0, self._pos, c)
        else:
            self._mine[:c.shape[0]].copy_(c)
            dist.all_gather_into_tensor(self._all.view(-1), self._mine, group=self.groups.fiber)
            for z, (o, l) in enumerate(self.slices):
                if self._pos is None:
                    self.spmm.vals[o:o + l].copy_(self._all[z, :l])
                else:
                    self.spmm.vals.index_copy_(0, self._pos[o:o + l], self._all[z, :l])
        self.spmm.values_changed()
        return self.spmm.run()
