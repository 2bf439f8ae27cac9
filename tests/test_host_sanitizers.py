"""The host library under AddressSanitizer + UndefinedBehaviorSanitizer.

A child process preloads the ASan runtime, selects the sanitized build of
csrc/host (SP3_HOST_SANITIZE=1) and drives the native host paths: file
formats, generators, partition + ownership + plans for several meshes, CPU
kernels, the simulators.  Any report makes the child exit non-zero.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]

CHILD = r"""
import os, sys, tempfile
import numpy as np, torch
from spcomm3d_b200.utils import native, generate, binfmt
from spcomm3d_b200.parallel.mesh import Mesh3D
from spcomm3d_b200.parallel.plan import build_all_plans
from spcomm3d_b200.parallel import virtual
from spcomm3d_b200.ops import local, oracle
assert native.host_sanitized() and native.build_host().name == "libsp3host_san.so"
mats = [generate.from_spec(s, seed=3) for s in
        ("uniform:300:200:5", "zipf:400:350:1.5:90", "rmat:9:8", "er:257:129:3")]
with tempfile.TemporaryDirectory() as d:
    for i, m in enumerate(mats):
        path = os.path.join(d, f"m{i}.bin")
        binfmt.write_bin(path, m)
        back = binfmt.read_bin(path)
        assert back.nnz == m.nnz and np.array_equal(back.rows, m.rows)
    mtx = os.path.join(d, "t.mtx")
    with open(mtx, "w") as f:
        f.write("%%MatrixMarket matrix coordinate real symmetric\n4 4 3\n1 1 1.5\n3 1 2.0\n4 2 -1\n")
    assert binfmt.read_mtx(mtx, mirror_diagonal=False).nnz == 5 and binfmt.read_mtx(mtx).nnz == 6
for m in mats:
    for meshstr in ("1x1x1", "2x2x1", "3x2x2", "1x4x2", "5x1x1"):
        mesh = Mesh3D.parse(meshstr)
        _, plans = build_all_plans(m, mesh, seed=1)
        assert sum(p.nnz for p in plans.values()) == m.nnz * mesh.Z
        p = plans[mesh.size - 1]
        k = 12
        A = generate.fill_rows(p.row.local_gids, k, 0, k, seed=2, stream=1)
        B = generate.fill_rows(p.col.local_gids, k, 0, k, seed=2, stream=2)
        A, B = torch.from_numpy(np.asarray(A, np.float32)), torch.from_numpy(np.asarray(B, np.float32))
        ri, ci = torch.from_numpy(p.rowidx), torch.from_numpy(p.colidx)
        vals = torch.from_numpy(p.vals).float()
        c = local.sddmm(ri, ci, vals, A, B)
        y = torch.zeros(p.row.n_local, k)
        local.spmm(torch.from_numpy(p.rowptr), ri, ci, vals, B, y, 0.0)
        assert torch.isfinite(c).all() and torch.isfinite(y).all()
    virtual.serial_sim(m, 3, 2, seed=1)
    virtual.count_excess(m, 2, 2, seed=1)
    virtual.count_empty(m)
print("sanitized host paths ok")
"""


def test_host_library_under_asan_ubsan():
    asan = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not asan or not os.path.isabs(asan) or not os.path.exists(asan):
        pytest.skip("no ASan runtime in this toolchain")
    env = dict(os.environ, SP3_HOST_SANITIZE="1", LD_PRELOAD=asan, PYTHONPATH=str(REPO),
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=97", UBSAN_OPTIONS="print_stacktrace=1",
               OMP_NUM_THREADS="4")
    res = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "sanitized host paths ok" in res.stdout
    assert "runtime error" not in res.stderr and "AddressSanitizer" not in res.stderr, res.stderr[-4000:]
