"""readDistribute: offline 2D pre-partitioner.

    readDistribute -x X -y Y [-o prefix] matrix.mtx|matrix.bin

Applies the seeded random round-robin row/column maps and writes one .bin
file per X x Y block (`prefix_x_y.bin`, global indices), so that a later run
can read its block directly.  The reference's tool of the same purpose
(tools/read_distribute_mm.cpp:81-127) writes one file holding block counts
followed by the triplets and truncates it by a size bug (:122); separate,
self-describing files avoid both.
"""
from __future__ import annotations

import argparse
import os
import sys

from ..parallel.mesh import Mesh3D
from ..parallel.partition import bucket_blocks, extract_block, make_maps
from ..utils import binfmt


def main(argv=None):
    ap = argparse.ArgumentParser(prog="readDistribute", description=__doc__.split("\n")[0])
    ap.add_argument("matrix")
    ap.add_argument("-x", type=int, required=True)
    ap.add_argument("-y", type=int, required=True)
    ap.add_argument("-o", dest="prefix", default=None)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    m = binfmt.read_mtx(args.matrix) if args.matrix.endswith(".mtx") else binfmt.read_bin(args.matrix)
    mesh = Mesh3D(args.x, args.y, 1)
    rowmap, colmap = make_maps(m.nrows, m.ncols, mesh, args.seed)
    offsets, perm = bucket_blocks(m, rowmap, colmap, mesh)
    prefix = args.prefix or os.path.splitext(args.matrix)[0]
    for x in range(args.x):
        for y in range(args.y):
            blk = extract_block(m, offsets, perm, mesh, x, y)
            path = f"{prefix}_{x}_{y}.bin"
            binfmt.write_bin(path, blk)
            print(f"{path}: {blk.nnz} nonzeros")


if __name__ == "__main__":
    main(sys.argv[1:])
