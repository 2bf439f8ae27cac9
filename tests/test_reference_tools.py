"""Compatibility with the reference's own serial programs, built unmodified
with its Makefile's commands (tools/read_convert_mm.cpp -> conv2bin,
miniapp/numCheckSeq.cpp): the `.bin` files are byte-identical and the SDDMM
checksum agrees to the digits the reference prints."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def ref_tools():
    sys.path.insert(0, str(REPO))
    from baseline import build_reference
    try:
        return build_reference.build_tools()
    except RuntimeError as e:
        pytest.skip(f"reference tools unavailable: {e}")


def _write_mtx(path, kind, nrows, ncols, entries):
    with open(path, "w") as f:
        f.write(f"%%MatrixMarket matrix coordinate {kind}\n% generated for the test\n")
        f.write(f"{nrows} {ncols} {len(entries)}\n")
        for e in entries:
            f.write(" ".join(str(x) for x in e) + "\n")


def _cases(tmp_path):
    rng = np.random.default_rng(11)
    out = []
    # general, real
    keys = rng.choice(300 * 200, 900, replace=False)
    ent = [(int(k // 200) + 1, int(k % 200) + 1, float(np.round(rng.random() * 4 - 2, 6))) for k in keys]
    p = tmp_path / "general.mtx"
    _write_mtx(p, "real general", 300, 200, ent)
    out.append(p)
    # symmetric (lower triangle incl. diagonal entries, which the reference mirrors too)
    ent = []
    for k in rng.choice(150 * 150, 500, replace=False):
        i, j = int(k // 150), int(k % 150)
        if i >= j:
            ent.append((i + 1, j + 1, float(np.round(rng.random(), 6))))
    p = tmp_path / "symm.mtx"
    _write_mtx(p, "real symmetric", 150, 150, ent)
    out.append(p)
    # pattern
    keys = rng.choice(120 * 90, 400, replace=False)
    p = tmp_path / "pattern.mtx"
    _write_mtx(p, "pattern general", 120, 90, [(int(k // 90) + 1, int(k % 90) + 1) for k in keys])
    out.append(p)
    return out


def test_bin_files_are_byte_identical_to_the_reference_converter(ref_tools, tmp_path):
    from spcomm3d_b200.utils import binfmt, native
    native_conv = native.build_tools()
    for mtx in _cases(tmp_path):
        ref_out = tmp_path / (mtx.stem + "_ref.bin")
        res = subprocess.run([str(ref_tools["conv2bin"]), "-o", str(ref_out), str(mtx)], capture_output=True, text=True)
        assert res.returncode == 0 and ref_out.exists(), res.stderr
        ours = tmp_path / (mtx.stem + "_ours.bin")
        binfmt.conv2bin(str(mtx), str(ours))
        assert ours.read_bytes() == ref_out.read_bytes(), mtx.name
        ours_native = tmp_path / (mtx.stem + "_native.bin")
        res = subprocess.run([str(native_conv), "-o", str(ours_native), str(mtx)], capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
        assert ours_native.read_bytes() == ref_out.read_bytes(), mtx.name


@pytest.mark.parametrize("k", [8, 32])
def test_sddmm_checksum_agrees_with_the_reference_oracle(ref_tools, tmp_path, k):
    for mtx in _cases(tmp_path):
        res = subprocess.run([str(ref_tools["numCheckSeq"]), "-k", str(k), str(mtx)], capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
        ref = float(res.stdout.strip().splitlines()[-1])
        res = subprocess.run([sys.executable, "-m", "spcomm3d_b200.cli.num_check_seq", "-k", str(k), str(mtx)],
                             capture_output=True, text=True, cwd=REPO)
        assert res.returncode == 0, res.stderr
        ours = float(res.stdout.strip().splitlines()[-1].rsplit("=", 1)[1])
        assert ours == pytest.approx(ref, rel=2e-5, abs=1e-12), (mtx.name, ours, ref)


@pytest.mark.parametrize("k", [8, 20])
def test_spmm_agrees_with_the_reference_loop(ref_tools, tmp_path, k):
    """The reference's SpMM loop (src/core_ops.cpp:24-35, behind baseline/ref_spmm_check.cpp) against our CPU
    kernel and the fp64 oracle on the same files, read by the respective readers."""
    import torch
    from spcomm3d_b200.ops import local, oracle
    from spcomm3d_b200.utils import binfmt
    for mtx in _cases(tmp_path):
        res = subprocess.run([str(ref_tools["spmm_check"]), str(k), str(mtx)], capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
        ref_sum, ref_sq = (float(x) for x in res.stdout.split())
        m = binfmt.read_mtx(str(mtx))
        X = (torch.arange(m.ncols, dtype=torch.float64) % 97)[:, None] / 100 + \
            torch.arange(k, dtype=torch.float64)[None, :] / 1000
        y_oracle = oracle.spmm_ref(m, X)
        order = np.lexsort((m.cols, m.rows))
        rows, cols, vals = m.rows[order], m.cols[order], m.vals[order]
        rowptr = np.zeros(m.nrows + 1, np.int64)
        np.cumsum(np.bincount(rows, minlength=m.nrows), out=rowptr[1:])
        Y = torch.zeros(m.nrows, k, dtype=torch.float64)
        local.spmm(torch.from_numpy(rowptr), torch.from_numpy(rows.astype(np.int32)),
                   torch.from_numpy(cols.astype(np.int32)), torch.from_numpy(vals), X, Y, 0.0)
        for y in (y_oracle, Y):
            assert float(y.sum()) == pytest.approx(ref_sum, rel=1e-9, abs=1e-9), mtx.name
            assert float((y * y).sum()) == pytest.approx(ref_sq, rel=1e-9), mtx.name
