"""Copies the reference sources to baseline/_ref (git-ignored) and builds the
timing driver against them with the shared-memory MPI subset of
baseline/mpi_shim.  Nothing in the reference tree is modified; `-include array`
supplies a header some of its files use without including
(src/comm_stats.cpp:45, src/dcomm_setup.cpp:27, src/distributed_comp.cpp:26).
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DST = HERE / "_ref"
REF_SOURCES = ["comm_setup.cpp", "comm_stats.cpp", "core_ops.cpp", "dcomm_setup.cpp", "distribute.cpp",
               "distributed_comp.cpp"]


def find_reference() -> Path | None:
    """The reference tree: the directory named by SP3_REFERENCE_DIR, else a checkout beside this repository
    (../reference), else the copy already made under baseline/_ref."""
    for cand in (os.environ.get("SP3_REFERENCE_DIR"), str(HERE.parent.parent / "reference"), str(REF_DST / "SpComm3D")):
        if cand and (Path(cand) / "src" / "core_ops.cpp").exists():
            return Path(cand)
    return None


def build(verbose=False) -> Path:
    """Returns the path of the built driver; raises RuntimeError with the reason otherwise."""
    dst = REF_DST / "SpComm3D"
    exe = REF_DST / "ref_driver"
    if not (dst / "src" / "core_ops.cpp").exists():
        src = find_reference()
        if src is None:
            raise RuntimeError("reference sources not found (set SP3_REFERENCE_DIR, or place them under baseline/_ref/SpComm3D)")
        REF_DST.mkdir(exist_ok=True)
        shutil.copytree(src, dst, dirs_exist_ok=True)
    inputs = [HERE / "ref_driver.cpp", HERE / "mpi_shim" / "mpi_shim.cpp", HERE / "mpi_shim" / "mpi.h"]
    if exe.exists() and all(exe.stat().st_mtime > p.stat().st_mtime for p in inputs):
        return exe
    cmd = ["g++", "-w", "--std=c++17", "-O3", "-include", "array", f"-I{dst / 'src'}", f"-I{HERE / 'mpi_shim'}",
           str(HERE / "ref_driver.cpp"), str(HERE / "mpi_shim" / "mpi_shim.cpp"),
           *[str(dst / "src" / s) for s in REF_SOURCES], "-o", str(exe), "-lrt", "-pthread"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("reference build failed: " + res.stderr[-600:].replace("\n", " | "))
    if verbose:
        print("built", exe)
    return exe


def build_tools() -> dict:
    """The reference's two serial programs, built with its Makefile's own commands (Makefile:23-27):
    {"conv2bin": path, "numCheckSeq": path}, plus "spmm_check": baseline/ref_spmm_check.cpp linked with the
    reference's SpMM loop.  Raises RuntimeError with the reason otherwise."""
    dst = REF_DST / "SpComm3D"
    if not (dst / "src" / "core_ops.cpp").exists():
        src = find_reference()
        if src is None:
            raise RuntimeError("reference sources not found")
        REF_DST.mkdir(exist_ok=True)
        shutil.copytree(src, dst, dirs_exist_ok=True)
    out = {}
    for name, cmd in (("conv2bin", ["g++", "-w", "-o", str(REF_DST / "ref_conv2bin"),
                                    str(dst / "tools" / "read_convert_mm.cpp"), f"-I{dst / 'src'}"]),
                      ("numCheckSeq", ["g++", "-w", "-O3", "-o", str(REF_DST / "ref_numCheckSeq"),
                                       str(dst / "miniapp" / "numCheckSeq.cpp"), str(dst / "src" / "core_ops.cpp"),
                                       f"-I{dst / 'src'}"]),
                      # the reference's SpMM loop and reader behind a few lines of our own (ref_spmm_check.cpp)
                      ("spmm_check", ["g++", "-w", "-O3", "-o", str(REF_DST / "ref_spmm_check"),
                                      str(HERE / "ref_spmm_check.cpp"), str(dst / "src" / "core_ops.cpp"),
                                      f"-I{dst / 'src'}"])):
        exe = Path(cmd[cmd.index("-o") + 1])
        if not exe.exists():
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"reference {name} build failed: " + res.stderr[-600:].replace("\n", " | "))
        out[name] = exe
    return out


if __name__ == "__main__":
    print(build(verbose=True))
    print(build_tools())
