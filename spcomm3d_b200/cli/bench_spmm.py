"""benchSpMM: distributed SpMM benchmark.

    benchSpMM [-k k1,k2,...] [-c Z] [-i iters] matrix.bin

Per k: the sparse instances and then the dense instance, `iters` iterations
each, two statistics lines per iteration (miniapp/bench_spmm.cpp:122-226).
"""
from __future__ import annotations

import sys

from ..models.dist_ops import DistSpMM
from ..utils import generate
from .bench_sddmm import run_instances
from .common import Runtime, base_parser


def main(argv=None):
    ap = base_parser("benchSpMM", __doc__.split("\n")[0])
    ap.add_argument("--normal", action="store_true", help="N(0,1) operands instead of the constant fill")
    args = ap.parse_args(argv)
    rt = Runtime(args)
    plan = rt.load_plan(args)
    xy = rt.mesh.xy_rank(*plan.coords[:2])

    def fill(op):
        kind = generate.FILL_NORMAL if args.normal else generate.FILL_CONST
        op.fill_owned(op.X_owned, plan.col.owned_gids, kind=kind, const=xy + 1, seed=args.seed, stream=2)

    run_instances(rt, plan, args, DistSpMM, ("fused", "sparseNRB", "sparse", "dense"), fill)
    rt.finish()


if __name__ == "__main__":
    main(sys.argv[1:])
