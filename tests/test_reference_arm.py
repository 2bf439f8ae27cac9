"""The reference build (unmodified sources + shared-memory MPI subset) and the
`--impl reference` arm of bench.py, on a tiny matrix."""
import json
import os
import subprocess
import sys

import pytest

from dist_utils import ROOT, free_port

sys.path.insert(0, ROOT)
from baseline import build_reference  # noqa: E402

pytestmark = pytest.mark.skipif(build_reference.find_reference() is None and
                                not (build_reference.REF_DST / "ref_driver").exists(),
                                reason="reference sources are not available")


def _last_json(text):
    lines = [l for l in text.splitlines() if l.startswith("{")]
    assert lines, text[-2000:]
    return json.loads(lines[-1])


def test_reference_arm_single_rank():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gen",
                          "uniform:600:500:6", "--k", "16", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    d = _last_json(out.stdout)
    assert d["impl"] == "reference" and "unavailable" not in d, d
    assert d["config"]["nnz"] == 3600 and d["config"]["mesh"] == "1x1x1" and d["value"] > 0
    assert d["steps"] == 2 and d["higher_is_better"] is False


def test_reference_arm_four_ranks_under_torchrun():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "bench.py"), "--impl", "reference",
           "--gpus", "4", "--gen", "uniform:600:500:6", "--k", "16", "--steps", "2", "--warmup", "1"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    d = _last_json(out.stdout)
    assert d["n_gpus"] == 4 and d["config"]["mesh"] == "2x2x1" and d["sddmm_ms"] > 0 and d["spmm_ms"] > 0
