"""benchSddmm: distributed SDDMM benchmark.

    benchSddmm [-k k1,k2,...] [-c Z] [-i iters] matrix.bin

For every k runs the instances "sparseNB" (here: the fused zero-staging
kernel, GPUs only), "sparseNRB", "sparse" and "dense", `iters` iterations
each, and prints the reference's two statistics lines (PRE, POST) per
iteration -- the programme of miniapp/bench_sddmm.cpp:122-268 /
miniapp/bench_both.cpp:122-266.  Operands are the constant `xy rank + 1` as in
the reference (bench_both.cpp:189-192) unless --normal is given.
"""
from __future__ import annotations

import sys

from ..models.dist_ops import DistSDDMM
from ..utils import generate, stats
from .common import Runtime, base_parser, klist


def run_instances(rt, plan, args, kernel_cls, default_variants, fill):
    for k in klist(args.klist):
        for variant in rt.variants(args, default_variants):
            rt.checkpoint()
            try:
                op = kernel_cls(plan, rt.groups, k, rt.dtype, rt.device, variant)
            except ValueError as e:
                rt.say(f"# skipping {variant} k={k}: {e}")
                continue
            fill(op)
            total = 0.0
            op.defer_status = True   # a kernel status is raised by close(), after every rank has let go
            try:
                for _ in range(args.iters):
                    rt.barrier()
                    op.run()
                    aggs = stats.report_iteration(op, rt.groups, rt.rank)
                    total += aggs["PRE"]["times"][stats.TIME_KEYS.index("total")]
                if args.json and rt.rank == 0:
                    print(stats.json_record(op, op.kernel, total / max(1, args.iters)))
            finally:
                op.close()
            del op


def main(argv=None):
    ap = base_parser("benchSddmm", __doc__.split("\n")[0])
    ap.add_argument("--normal", action="store_true", help="N(0,1) operands instead of the constant fill")
    args = ap.parse_args(argv)
    rt = Runtime(args)
    plan = rt.load_plan(args)
    xy = rt.mesh.xy_rank(*plan.coords[:2])

    def fill(op):
        kind = generate.FILL_NORMAL if args.normal else generate.FILL_CONST
        op.fill_owned(op.A_owned, plan.row.owned_gids, kind=kind, const=xy + 1, seed=args.seed, stream=1)
        op.fill_owned(op.B_owned, plan.col.owned_gids, kind=kind, const=xy + 1, seed=args.seed, stream=2)

    run_instances(rt, plan, args, DistSDDMM, ("fused", "sparseNRB", "sparse", "dense"), fill)
    rt.finish()


if __name__ == "__main__":
    main(sys.argv[1:])
