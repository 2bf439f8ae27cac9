"""Builds and loads the two native libraries of the framework.

* ``libsp3host.so``  -- C++17 host code (``csrc/host``): file formats,
  generators, partitioning, ownership, CSR ordering, CPU kernels, simulators.
* ``libsp3cuda.so``  -- hand-written sm_100a CUDA kernels (``csrc/kernels``).

Both are plain ``extern "C"`` libraries called through :mod:`ctypes` with raw
pointers (``tensor.data_ptr()`` / ``ndarray.ctypes``) and, for kernels, the raw
handle of the current CUDA stream.  They are built in-tree
(``spcomm3d_b200/_lib``) so the binaries travel with a source snapshot; a
content stamp beside each library decides whether a rebuild is needed.

The reference is built by a three-line Makefile with ``mpic++``
(Makefile:1-3); there is no equivalent of a loader there.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parents[2]
CSRC = REPO / "csrc"
LIBDIR = Path(__file__).resolve().parents[1] / "_lib"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

_TYPES = {
    "i32": ctypes.c_int32, "u32": ctypes.c_uint32, "i64": ctypes.c_int64, "u64": ctypes.c_uint64,
    "int": ctypes.c_int, "f32": ctypes.c_float, "f64": ctypes.c_double, "p": ctypes.c_void_p,
    "s": ctypes.c_char_p,
}

# name -> (restype, "argtypes")
HOST_SIGS = {
    "sp3_bin_read_header": ("int", "s p p p"),
    "sp3_bin_read_range": ("int", "s u64 u64 p p p p"),
    "sp3_bin_write": ("int", "s u32 u32 u64 p p p p"),
    "sp3_mm_read_header": ("int", "s p p p p p"),
    "sp3_mm_read": ("int", "s u64 int p p p p"),
    "sp3_mm_write": ("int", "s u64 u64 u64 p p p"),
    "sp3_gen_fixed_degree": ("int", "u64 u64 u32 u64 p p p"),
    "sp3_gen_degrees": ("int", "u64 int f64 u32 u32 u64 p"),
    "sp3_gen_from_rowptr": ("int", "u64 u64 p u64 p p p"),
    "sp3_gen_from_rowptr_block": ("int", "u64 u64 p u64 p i32 p i32 p p p p"),
    "sp3_gen_rmat_keys": ("int", "u32 u64 f64 f64 f64 u64 p"),
    "sp3_sort_unique_u64": ("i64", "p u64"),
    "sp3_keys_to_coo": ("int", "p u64 u64 p p p"),
    "sp3_fill_rows_f64": ("int", "p u64 u64 u64 u64 u64 int f64 u64 u64 p"),
    "sp3_fill_rows_f32": ("int", "p u64 u64 u64 u64 u64 int f64 u64 u64 p"),
    "sp3_rr_map": ("int", "u64 u32 u64 u64 p"),
    "sp3_bucket_blocks": ("int", "u64 p p p p u32 u32 p p"),
    "sp3_touch_masks": ("int", "u64 p p p p p p"),
    "sp3_assign_owners": ("int", "u64 p p u32 u32 int u64 u64 p p p"),
    "sp3_csr_order": ("int", "u64 p p u64 p p"),
    "sp3_remap_u32": ("int", "u64 p p u64 p"),
    "sp3_count_empty": ("int", "u64 p p u64 u64 p p"),
    "sp3_cpu_sddmm_f32": ("int", "i64 p p p p i64 p i64 i64 p"),
    "sp3_cpu_sddmm_f64": ("int", "i64 p p p p i64 p i64 i64 p"),
    "sp3_cpu_spmm_f32": ("int", "i64 p p p p i64 i64 f32 p i64"),
    "sp3_cpu_spmm_f64": ("int", "i64 p p p p i64 i64 f64 p i64"),
    "sp3_cpu_rows_f32": ("int", "int i64 p p i64 p i64 i64"),
    "sp3_cpu_rows_f64": ("int", "int i64 p p i64 p i64 i64"),
    "sp3_serial_sim": ("int", "u64 p p u64 u64 u32 u32 u64 int int p"),
    "sp3_count_excess": ("int", "u64 p p u64 u64 u32 u32 u64 p"),
}

ERRORS = {-1: "I/O error", -2: "bad file format", -3: "index out of range", -4: "bad argument",
          -5: "capacity too small"}


class NativeError(RuntimeError):
    pass


def _sources(sub: str, exts) -> list[Path]:
    d = CSRC / sub
    return sorted(p for p in d.iterdir() if p.suffix in exts)


def _stamp(files, flags) -> str:
    h = hashlib.sha256()
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    # flags enter the stamp with the checkout path removed, so a snapshot of
    # the tree copied elsewhere does not look stale
    h.update(" ".join(flags).replace(str(REPO), ".").encode())
    return h.hexdigest()


def _build(lib: Path, srcs, hdrs, cmd, force=False, verbose=False) -> bool:
    """Runs `cmd` when the stamp of sources+flags differs from the stored one."""
    LIBDIR.mkdir(exist_ok=True)
    stamp_file = lib.with_suffix(".stamp")
    want = _stamp(list(srcs) + list(hdrs), cmd)
    if not force and lib.exists() and stamp_file.exists() and stamp_file.read_text() == want:
        return False
    with open(LIBDIR / ".build.lock", "w") as lk:
        fcntl.flock(lk, fcntl.LOCK_EX)
        if not force and lib.exists() and stamp_file.exists() and stamp_file.read_text() == want:
            return False
        tmp = lib.with_suffix(f".tmp{os.getpid()}.so")
        full = cmd + ["-o", str(tmp)] + [str(s) for s in srcs]
        if verbose:
            print("[spcomm3d_b200] building", lib.name, file=sys.stderr)
        res = subprocess.run(full, capture_output=True, text=True)
        if res.returncode != 0:
            raise NativeError(f"build of {lib.name} failed:\n{' '.join(full)}\n{res.stdout}\n{res.stderr}")
        if verbose and res.stderr:
            print(res.stderr, file=sys.stderr)
        os.replace(tmp, lib)
        stamp_file.write_text(want)
    return True


def host_sanitized() -> bool:
    """SP3_HOST_SANITIZE=1 selects a build of the host library with AddressSanitizer and
    UndefinedBehaviorSanitizer (libsp3host_san.so).  The process must have the ASan runtime loaded first
    (LD_PRELOAD of `gcc -print-file-name=libasan.so`); tests/test_host_sanitizers.py runs such a child."""
    return os.environ.get("SP3_HOST_SANITIZE", "0") == "1"


def host_build_cmd():
    cmd = ["g++", "-std=c++17", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden", f"-I{CSRC / 'host'}"]
    if host_sanitized():
        return cmd + ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
                      "-fno-sanitize-recover=undefined"]
    return cmd + ["-O3"]


def cuda_build_cmd(verbose_ptxas=False):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo", *NVCC_ARCH, "-shared", "-Xcompiler", "-fPIC",
           "-Xcompiler", "-fvisibility=hidden", f"-I{CSRC / 'kernels'}"]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("SP3_NVCC_DEFS", "").split()  # e.g. "-DSP3_SDDMM_MINB=4" for tuning builds
    return cmd


def build_host(force=False, verbose=False) -> Path:
    lib = LIBDIR / ("libsp3host_san.so" if host_sanitized() else "libsp3host.so")
    _build(lib, _sources("host", {".cpp"}), _sources("host", {".hpp"}), host_build_cmd(), force, verbose)
    return lib


def build_cuda(force=False, verbose=False) -> Path:
    """Compiles every .cu of csrc/kernels for sm_100a (one nvcc process per
    file, in parallel) and links them into libsp3cuda.so."""
    lib = LIBDIR / "libsp3cuda.so"
    srcs = _sources("kernels", {".cu"})
    hdrs = _sources("kernels", {".cuh", ".h"})
    cmd = cuda_build_cmd()
    LIBDIR.mkdir(exist_ok=True)
    stamp_file = lib.with_suffix(".stamp")
    want = _stamp(list(srcs) + list(hdrs), cmd)
    if not force and lib.exists() and stamp_file.exists() and stamp_file.read_text() == want:
        return lib
    with open(LIBDIR / ".build.lock", "w") as lk:
        fcntl.flock(lk, fcntl.LOCK_EX)
        if not force and lib.exists() and stamp_file.exists() and stamp_file.read_text() == want:
            return lib
        if verbose:
            print("[spcomm3d_b200] building", lib.name, file=sys.stderr)
        objdir = LIBDIR / "obj"
        objdir.mkdir(exist_ok=True)
        compile_cmd = [c for c in cmd if c != "-shared"] + ["-c"]

        def one(src):
            obj = objdir / (src.stem + ".o")
            res = subprocess.run(compile_cmd + ["-o", str(obj), str(src)], capture_output=True, text=True)
            if res.returncode != 0:
                raise NativeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
            return obj

        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=len(srcs)) as ex:
            objs = list(ex.map(one, srcs))
        tmp = lib.with_suffix(f".tmp{os.getpid()}.so")
        res = subprocess.run(cmd + ["-o", str(tmp)] + [str(o) for o in objs], capture_output=True, text=True)
        if res.returncode != 0:
            raise NativeError(f"link of {lib.name} failed:\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, lib)
        stamp_file.write_text(want)
    return lib


def build_tools(force=False, verbose=False) -> Path:
    """Standalone native conv2bin executable (links the host sources directly)."""
    exe = LIBDIR / "conv2bin"
    srcs = [CSRC / "tools" / "conv2bin.cpp", CSRC / "host" / "io.cpp"]
    cmd = ["g++", "-std=c++17", "-O3", f"-I{CSRC / 'host'}"]
    _build(exe, srcs, _sources("host", {".hpp"}), cmd, force, verbose)
    # row-gather throughput probe (vector loads against bulk copies), see its header
    gb = LIBDIR / "gather_bench"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    _build(gb, [CSRC / "tools" / "gather_bench.cu"], [CSRC / "kernels" / "sp3_async.cuh", CSRC / "kernels" / "sp3_cuda.cuh"],
           [nvcc, "-std=c++17", "-O3", "-lineinfo", *NVCC_ARCH, f"-I{CSRC / 'kernels'}"], force, verbose)
    return exe


def _bind(lib, sigs):
    for name, (res, args) in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.restype = _TYPES[res]
        fn.argtypes = [_TYPES[a] for a in args.split()]


_host = None
_cuda = None


def host():
    """The host library, built on first use."""
    global _host
    if _host is None:
        path = build_host()
        _host = ctypes.CDLL(str(path))
        _bind(_host, HOST_SIGS)
    return _host


def cuda():
    """The CUDA kernel library.  Raises if it cannot be built or loaded: GPU
    code paths never fall back silently to another implementation."""
    global _cuda
    if _cuda is None:
        # SP3_CUDA_LIB: load this build of the kernel library instead (tuning builds with other compile-time knobs)
        path = os.environ.get("SP3_CUDA_LIB") or build_cuda()
        _cuda = ctypes.CDLL(str(path))
        from .cuda_sigs import CUDA_SIGS
        _bind(_cuda, CUDA_SIGS)
    return _cuda


def ptr(x):
    """Raw pointer of a numpy array / torch tensor / None."""
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        if not x.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be C-contiguous")
        return x.ctypes.data
    return x.data_ptr()  # torch tensor


def check(rc: int, what: str):
    if rc != 0:
        raise NativeError(f"{what}: {ERRORS.get(rc, f'error {rc}')}")
