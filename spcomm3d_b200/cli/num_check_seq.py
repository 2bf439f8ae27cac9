"""numCheckSeq: serial SDDMM checksum.

    numCheckSeq [-k k] matrix.mtx|matrix.bin

Fills A[i, :] = B[i, :] = i / 1000, runs SDDMM on one process and prints the
sum of the result values, like miniapp/numCheckSeq.cpp:101-134.
"""
from __future__ import annotations

import argparse
import sys

import numpy as np

from ..ops import oracle
from ..utils import binfmt, generate


def checksum_of(path_or_matrix, k: int) -> float:
    m = path_or_matrix
    if isinstance(m, str):
        m = binfmt.read_mtx(m) if m.endswith(".mtx") else binfmt.read_bin(m)
    A = generate.fill_rows(np.arange(m.nrows), k, 0, k, kind=generate.FILL_GID_OVER_1000, dtype=np.float64)
    B = generate.fill_rows(np.arange(m.ncols), k, 0, k, kind=generate.FILL_GID_OVER_1000, dtype=np.float64)
    return oracle.checksum(oracle.sddmm_ref(m, A, B))


def main(argv=None):
    ap = argparse.ArgumentParser(prog="numCheckSeq", description=__doc__.split("\n")[0])
    ap.add_argument("matrix")
    ap.add_argument("-k", type=int, default=32)
    args = ap.parse_args(argv)
    print(f"Numerical sum = {checksum_of(args.matrix, args.k):.12g}")


if __name__ == "__main__":
    main(sys.argv[1:])
