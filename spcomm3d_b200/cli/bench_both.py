"""benchBoth: SpMM and SDDMM back to back on one matrix (GNN-layer style).

    benchBoth [-k k1,k2,...] [-c Z] [-i iters] matrix.bin

Order per k, as intended by miniapp/main_combined.cpp:165-281: sparse SpMM,
sparse SDDMM, dense SpMM, dense SDDMM.  `--chain` additionally runs the
attention-style chain (SDDMM scores used as the SpMM values).
"""
from __future__ import annotations

import sys

from ..models.dist_ops import DistSDDMM, DistSpMM
from ..models.layer import GatLayer
from ..utils import generate, stats
from .common import Runtime, base_parser, klist


def main(argv=None):
    ap = base_parser("benchBoth", __doc__.split("\n")[0])
    ap.add_argument("--chain", action="store_true")
    args = ap.parse_args(argv)
    rt = Runtime(args)
    plan = rt.load_plan(args)
    xy = rt.mesh.xy_rank(*plan.coords[:2])
    sparse_variant = rt.variants(args, ("fused",) if rt.device.type == "cuda" else ("sparseNRB",))
    sparse_variant = (sparse_variant or ["sparseNRB"])[0]
    for k in klist(args.klist):
        for variant in (sparse_variant, "dense"):
            for cls in (DistSpMM, DistSDDMM):
                op = cls(plan, rt.groups, k, rt.dtype, rt.device, variant)
                for name, side in (("A_owned", plan.row), ("B_owned", plan.col), ("X_owned", plan.col)):
                    if hasattr(op, name):
                        op.fill_owned(getattr(op, name), side.owned_gids, kind=generate.FILL_CONST, const=xy + 1)
                for _ in range(args.iters):
                    rt.barrier()
                    op.run()
                    stats.report_iteration(op, rt.groups, rt.rank)
                del op
        if args.chain:
            layer = GatLayer(plan, rt.groups, k, rt.dtype, rt.device, sparse_variant)
            layer.sddmm.fill_owned(layer.sddmm.A_owned, plan.row.owned_gids, seed=args.seed, stream=1)
            layer.sddmm.fill_owned(layer.sddmm.B_owned, plan.col.owned_gids, seed=args.seed, stream=2)
            layer.spmm.fill_owned(layer.spmm.X_owned, plan.col.owned_gids, seed=args.seed, stream=2)
            for _ in range(args.iters):
                rt.barrier()
                y = layer.run()
            rt.say(f"# chain SDDMM->SpMM k={k}: local checksum {float(y.double().sum()):.6f}")
    rt.finish()


if __name__ == "__main__":
    main(sys.argv[1:])
