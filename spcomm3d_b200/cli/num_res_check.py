"""numResCheck: distributed SDDMM (and SpMM) checksum against the serial one.

    numResCheck [-k k] [-c Z] [--variant v] matrix.bin

Operand rows are filled by *global* id (row i = i / 1000), one distributed
SDDMM runs per variant, every rank prints the sum of the values it owns and
rank 0 the global sum, to be compared with numCheckSeq
(miniapp/numResCheck_sddmm_parallel.cpp:181-195).  Unlike the reference,
non-owned rows are poisoned with NaN before the run, so a broken gather
cannot pass, and SpMM is checked too.
"""
from __future__ import annotations

import sys


from ..models.dist_ops import DistSDDMM, DistSpMM
from ..utils import generate
from .common import Runtime, base_parser, klist


def main(argv=None):
    ap = base_parser("numResCheck", __doc__.split("\n")[0])
    args = ap.parse_args(argv)
    rt = Runtime(args)
    plan = rt.load_plan(args)
    results = {}
    for k in klist(args.klist):
        for variant in rt.variants(args, ("sparseNRB", "dense")):
            for cls in (DistSDDMM, DistSpMM):
                op = cls(plan, rt.groups, k, rt.dtype, rt.device, variant)
                for name, side in (("A_owned", plan.row), ("B_owned", plan.col), ("X_owned", plan.col)):
                    if hasattr(op, name):
                        op.fill_owned(getattr(op, name), side.owned_gids, kind=generate.FILL_GID_OVER_1000)
                op.poison_unowned()
                mine = op.run().double().sum().reshape(1)
                print(f"Numerical sum at p{rt.rank} = {float(mine):.12g}")
                if rt.world > 1:
                    import torch.distributed as dist
                    t = mine.to(rt.device)
                    dist.all_reduce(t)
                    mine = t.cpu()
                results[(op.kernel, variant, k)] = float(mine)
                rt.say(f"Global numerical sum ({variant} {op.kernel}, k={k}) = {float(mine):.12g}")
    rt.finish()
    return results


if __name__ == "__main__":
    main(sys.argv[1:])
