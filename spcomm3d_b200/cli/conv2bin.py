"""conv2bin: MatrixMarket -> binary converter.

    conv2bin [-o out.bin] [-d] [-j JOBS] in.mtx [more.mtx ...]

Same output as the reference tool (tools/read_convert_mm.cpp:81-145); the
native executable built from csrc/tools/conv2bin.cpp does the same without
Python.  `-z` is accepted and ignored, as in the reference.  Several inputs
are converted in one call, `-j` of them at a time: the job of the reference's
batch scripts (scripts/convert2bin.sh, scripts/convert2bin-par.sh).
"""
from __future__ import annotations

import argparse
import sys

from ..utils import binfmt


def main(argv=None):
    ap = argparse.ArgumentParser(prog="conv2bin", description=__doc__.split("\n")[0])
    ap.add_argument("mtx", nargs="+")
    ap.add_argument("-j", dest="jobs", type=int, default=1)
    ap.add_argument("-o", dest="out", default=None)
    ap.add_argument("-z", dest="z", default=None, help="ignored")
    ap.add_argument("-d", dest="dedup_diag", action="store_true",
                    help="store diagonal entries of symmetric matrices once")
    args = ap.parse_args(argv)
    if args.out and len(args.mtx) > 1:
        ap.error("-o needs a single input")

    def one(path):
        out = binfmt.conv2bin(path, args.out, mirror_diagonal=not args.dedup_diag)
        nr, nc, nnz = binfmt.read_bin_header(out)
        return f"{path}: {nr} x {nc}, {nnz} nonzeros -> {out}"

    if args.jobs > 1 and len(args.mtx) > 1:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(args.jobs) as ex:
            for line in ex.map(one, args.mtx):
                print(line)
    else:
        for path in args.mtx:
            print(one(path))


if __name__ == "__main__":
    main(sys.argv[1:])
