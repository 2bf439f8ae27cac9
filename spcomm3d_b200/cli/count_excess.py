"""countExcess / countEmptyRows: memory-excess and empty-line counters.

    countExcess [-n P] matrix      dense rows stored by the sparsity-agnostic
                                   method minus rows actually touched, summed
                                   over the ranks (miniapp/countExcess.cpp:135-155)
    countExcess --empty matrix     rows and columns without nonzeros
                                   (tools/countEmptyRows.cpp:80-92)
"""
from __future__ import annotations

import argparse
import sys

from ..parallel import virtual
from ..utils import binfmt


def main(argv=None):
    ap = argparse.ArgumentParser(prog="countExcess", description=__doc__.split("\n")[0])
    ap.add_argument("matrix")
    ap.add_argument("-n", dest="P", type=int, default=64)
    ap.add_argument("--empty", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    m = binfmt.read_mtx(args.matrix) if args.matrix.endswith(".mtx") else binfmt.read_bin(args.matrix)
    if args.empty:
        er, ec = virtual.count_empty(m)
        print(f"{m.name} empty rows {er} of {m.nrows}, empty cols {ec} of {m.ncols}")
        return
    X, Y = virtual.find_xy(args.P)
    r = virtual.count_excess(m, X, Y, seed=args.seed)
    print(f"{m.name} {args.P} {int(r['stored_rows'])} {int(r['touched_rows'])} {int(r['excess_rows'])}")


if __name__ == "__main__":
    main(sys.argv[1:])
