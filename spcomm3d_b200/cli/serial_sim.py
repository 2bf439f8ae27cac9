"""serialSim: communication volumes on virtual processor meshes, no ranks needed.

    serialSim [-n P1,P2,...] [-i dim -d density | -m matrix] [--mode sddmm|spmm_pre|spmm_post]

Without -m a square matrix of `dim` rows with `dim^2 * density` distinct
random nonzeros is generated.  For every P the most square X x Y is used and
two lines are printed: `S` (sparsity-aware plan) and `B` (whole-slab
broadcast), each with avg/max send/recv messages and dense rows
(miniapp/serialSim.cpp:227-252).  Defaults sweep P = 64 ... 32768 like the
reference (serialSim.cpp:285).
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
    args = ap.parse_args(argv)
    if args.matrix:
        m = binfmt.read_mtx(args.matrix) if args.matrix.endswith(".mtx") else binfmt.read_bin(args.matrix)
    else:
        m = CooMatrix.random_unique(args.dim, args.dim, int(args.dim * args.dim * args.density), seed=args.seed)
        m.name = f"random_{args.dim}_{args.density:g}"
    for P in (int(t) for t in args.plist.split(",")):
        X, Y = virtual.find_xy(P)
        res = virtual.serial_sim(m, X, Y, seed=args.seed, policy=args.policy, mode=args.mode)
        print(virtual.sim_line("S", m, P, res["sparse"]))
        print(virtual.sim_line("B", m, P, res["dense"]))


if __name__ == "__main__":
    main(sys.argv[1:])
