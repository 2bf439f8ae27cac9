"""emulate: all ranks of a mesh on ONE GPU, phase by phase.

    python -m spcomm3d_b200.cli.emulate --gen rmat:20:16 -k 128 --mesh 2x2x2

Builds every rank's plan and fused op in this process (heaps are local
allocations, "peer" addresses are ordinary device pointers), runs the three
kernel phases of all ranks in lock step and reports, for one rank, the device
time of its MAIN phase (pull + compute + push) next to the plain local kernel
on the same block.  No launch ever waits for a later launch.  This is how the
fused kernels are checked and profiled (one GPU, `ncu -k regex:fused_`) when
only one device is at hand; the reference's closest tool is its serial
simulator, which counts volumes but executes nothing
(miniapp/serialSim.cpp:109-252).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..models.dist_ops import DistSDDMM, DistSpMM
from ..ops import cuda_ops, local
from ..ops.fused import PH_MAIN, PH_START, FusedSDDMM, FusedSpMM, run_lockstep
from ..parallel.mesh import Mesh3D, split_k
from ..parallel.plan import build_all_plans
from ..parallel.symm import LocalFabric
from ..utils import generate


def _time(fn, n):
    for _ in range(2):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n


def main(argv=None):
    ap = argparse.ArgumentParser(prog="emulate", description=__doc__.split("\n")[0])
    ap.add_argument("--gen", required=True)
    ap.add_argument("-k", type=int, default=128)
    ap.add_argument("--mesh", default="2x2x2")
    ap.add_argument("--rank", type=int, default=0, help="rank whose MAIN phase is timed")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--only", default=None, choices=["sddmm", "spmm"])
    ap.add_argument("--no-overlap", action="store_true", help="SDDMM: compute only after all pulls (no reordering)")
    args = ap.parse_args(argv)
    mesh = Mesh3D.parse(args.mesh)
    m = generate.from_spec(args.gen, seed=args.seed)
    _, plans = build_all_plans(m, mesh, seed=args.seed)
    fabric = LocalFabric(mesh.size)
    kl = [split_k(args.k, mesh.Z, plans[r].coords[2])[1] for r in range(mesh.size)]
    for cls, F in ((DistSDDMM, FusedSDDMM), (DistSpMM, FusedSpMM)):
        if args.only and args.only != cls.kernel:
            continue
        kw = {"overlap": False} if (args.no_overlap and cls is DistSDDMM) else {}
        heaps = fabric.heaps([F.region_sizes(plans[r], kl[r]) for r in range(mesh.size)])
        ops = [cls(plans[r], None, args.k, torch.float32, "cuda", "fused", heap=heaps[r], timeout_s=5.0, **kw)
               for r in range(mesh.size)]
        for op in ops:
            for name, side, st in (("A_owned", op.plan.row, 1), ("B_owned", op.plan.col, 2),
                                   ("X_owned", op.plan.col, 2)):
                if hasattr(op, name):
                    op.fill_owned(getattr(op, name), side.owned_gids, seed=args.seed, stream=st)
        fs = [op._fused for op in ops]
        largs = [(op.Y_owned, 0.0) for op in ops] if cls is DistSpMM else [()] * len(ops)
        run_lockstep(fs, largs)
        f0, a0, p = fs[args.rank], largs[args.rank], ops[args.rank].plan

        def starts():
            for f, a in zip(fs, largs):
                f.launch(*a, phases=PH_START, new_epoch=True)

        def starts_and_main():
            starts()
            f0.launch(*a0, phases=PH_MAIN, new_epoch=False)

        t_main = _time(starts_and_main, args.steps) - _time(starts, args.steps)
        starts_and_main()
        in_kernel = f0.phase_ms()["main"]  # globaltimer stamps inside that last MAIN launch
        k0 = kl[args.rank]
        o = ops[args.rank]
        if cls is DistSDDMM:
            A = torch.randn(p.row.n_local, k0, device="cuda")
            B = torch.randn(p.col.n_local, k0, device="cuda")
            out = torch.empty(p.nnz, device="cuda")
            t_loc = _time(lambda: local.sddmm(o.rowidx, o.colidx, o.vals, A, B, out), args.steps)
        else:
            X = torch.randn(p.col.n_local, k0, device="cuda")
            Y = torch.zeros(p.row.n_local, k0, device="cuda")
            sch = cuda_ops.SpmmSchedule(o.rowptr)
            t_loc = _time(lambda: local.spmm(o.rowptr, o.rowidx, o.colidx, o.vals, X, Y, 0.0, sch), args.steps)
        run_lockstep(fs, largs)  # leave every rank in a consistent epoch
        for f in fs:
            f.check()
        print(json.dumps({"mesh": str(mesh), "kernel": cls.kernel, "rank": args.rank, "nnz_rank": p.nnz, "k_loc": k0,
                          "rows_pulled": p.col.n_recv, "rows_remote_rowside": p.row.n_recv,
                          "fused_main_ms": round(t_main, 4), "fused_main_in_kernel_ms": round(in_kernel, 4), "local_kernel_ms": round(t_loc, 4)}))
        del ops, fs, heaps


if __name__ == "__main__":
    main(sys.argv[1:])
