"""serialSim: communication volumes on virtual processor meshes, no ranks needed.

    serialSim [-n P1,P2,...] [-i dim -d density | -m matrix] [--mode sddmm|spmm_pre|spmm_post]

Without -m a square matrix of `dim` rows with `dim^2 * density` distinct
random nonzeros is generated.  For every P the most square X x Y is used and
two lines are printed: `S` (sparsity-aware plan) and `B` (whole-slab
broadcast), each with avg/max send/recv messages and dense rows
(miniapp/serialSim.cpp:227-252).  Defaults sweep P = 64 ... 32768 like the
reference (serialSim.cpp:285).

`--ref-format` prints the reference's own line layout (`name rows cols nnz N
XxYxZ f c S|B ...`), with N the total rank count including the Z layers given
by -c and its X <= Y mesh choice, so that post-processing written for the
reference reads these lines.  `--density-sweep` repeats the run for the
densities 1e-7, 1e-6, ..., 1e-3 on a generated matrix named SYNTH, which is the
reference's fixed programme (serialSim.cpp:278-287).
"""
from __future__ import annotations

import argparse
import sys

from ..parallel import virtual
from ..utils import binfmt
from ..utils.sparse import CooMatrix


def main(argv=None):
    ap = argparse.ArgumentParser(prog="serialSim", description=__doc__.split("\n")[0])
    ap.add_argument("-n", dest="plist", default="64,128,256,512,1024,2048,4096,8192,16384,32768")
    ap.add_argument("-i", dest="dim", type=int, default=100000)
    ap.add_argument("-d", dest="density", type=float, default=1e-4)
    ap.add_argument("-m", dest="matrix", default=None)
    ap.add_argument("--mode", default="sddmm", choices=list(virtual.MODES))
    ap.add_argument("--policy", default="random", choices=["respect_comm", "random"],
                    help="owner choice; the reference simulator uses the round-robin scheme")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("-k", dest="f", type=int, default=32, help="inner dimension (printed; volumes are in dense rows)")
    ap.add_argument("-c", dest="Z", type=int, default=1, help="Z layers: the plane that is simulated has P / Z ranks")
    ap.add_argument("--ref-format", action="store_true", help="print lines in the reference's layout")
    ap.add_argument("--density-sweep", action="store_true",
                    help="generated matrices at densities 1e-7 ... 1e-3 instead of one -d (name SYNTH)")
    args = ap.parse_args(argv)
    plist = [int(t) for t in args.plist.split(",")]
    if args.matrix:
        m = binfmt.read_mtx(args.matrix) if args.matrix.endswith(".mtx") else binfmt.read_bin(args.matrix)
        matrices = [m]
    else:
        densities = [10.0 ** e for e in range(-7, -2)] if args.density_sweep else [args.density]
        matrices = []
        for d in densities:
            m = CooMatrix.random_unique(args.dim, args.dim, int(args.dim * args.dim * d), seed=args.seed)
            m.name = "SYNTH" if args.density_sweep else f"random_{args.dim}_{d:g}"
            matrices.append(m)
    for m in matrices:
        for P in plist:
            if P % args.Z:
                print(f"# skipping P={P}: not a multiple of Z={args.Z}", file=sys.stderr)
                continue
            plane = P // args.Z
            X, Y = virtual.find_xy_ref(plane) if args.ref_format else virtual.find_xy(plane)
            res = virtual.serial_sim(m, X, Y, seed=args.seed, policy=args.policy, mode=args.mode,
                                     dense_as_messages=args.ref_format)
            if args.ref_format:
                print(virtual.sim_line_ref("S", m, P, X, Y, args.Z, args.f, res["sparse"]))
                print(virtual.sim_line_ref("B", m, P, X, Y, args.Z, args.f, res["dense"]))
            else:
                print(virtual.sim_line("S", m, P, res["sparse"]))
                print(virtual.sim_line("B", m, P, res["dense"]))


if __name__ == "__main__":
    main(sys.argv[1:])
