"""conv2bin: MatrixMarket -> binary converter.

    conv2bin [-o out.bin] [-d] in.mtx

Same output as the reference tool (tools/read_convert_mm.cpp:81-145); the
native executable built from csrc/tools/conv2bin.cpp does the same without
Python.  `-z` is accepted and ignored, as in the reference.
"""
from __future__ import annotations

import argparse
import sys

from ..utils import binfmt


def main(argv=None):
    ap = argparse.ArgumentParser(prog="conv2bin", description=__doc__.split("\n")[0])
    ap.add_argument("mtx")
    ap.add_argument("-o", dest="out", default=None)
    ap.add_argument("-z", dest="z", default=None, help="ignored")
    ap.add_argument("-d", dest="dedup_diag", action="store_true",
                    help="store diagonal entries of symmetric matrices once")
    args = ap.parse_args(argv)
    out = binfmt.conv2bin(args.mtx, args.out, mirror_diagonal=not args.dedup_diag)
    nr, nc, nnz = binfmt.read_bin_header(out)
    print(f"{args.mtx}: {nr} x {nc}, {nnz} nonzeros -> {out}")


if __name__ == "__main__":
    main(sys.argv[1:])
