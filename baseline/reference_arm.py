"""`bench.py --impl reference`: the unmodified reference, timed on the machine the bench runs on.

The reference (nfabubaker/SpComm3D) is C++ + MPI for CPUs.  It is not a Python
package (`pip install` of its tree fails: no setup.py / pyproject.toml), and
no MPI is installed, so its sources are copied to baseline/_ref and compiled,
unchanged, against the shared-memory MPI subset in baseline/mpi_shim together
with a small timing driver (baseline/ref_driver.cpp) that calls the
reference's own public functions in the order its benchmarks do.  One shim
rank runs per launched process (N ranks for --gpus N), on the host CPUs: the
reference has no GPU code.

Same matrix (generator spec + seed), same k, same mesh rule (Z fixed, X >= Y
balanced) as our arm; fp64, the reference's only value type.  The value is
best-of-its-SDDMM-variants + SpMM, milliseconds per iteration, max over ranks;
metric and unit strings are those of our arm.  Its operands live in host
memory and so does its result, so the same number is also its end-to-end
value.  --steps and --warmup are honoured up to a wall-clock allowance per
kernel (SP3_REF_BUDGET_S, default 150 s: a step is about 20 s of CPU time on
one rank for the headline matrix); the JSON line states the counts that ran
and, when the allowance cut them, says so in `config.steps_cap`.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

BUDGET_S = float(os.environ.get("SP3_REF_BUDGET_S", "150"))


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}))


def run(args, metric: str, unit: str):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    job = os.environ.get("MASTER_PORT", str(os.getppid()))
    tmp = Path(os.environ.get("TMPDIR", "/tmp")) / f"sp3_ref_{job}"
    ready, failed = tmp / "READY", tmp / "FAILED"
    steps, warmup = args.steps, args.warmup
    # same Z as our arm's default mesh; the reference then balances X >= Y itself (MPI_Dims_create)
    default_z = {1: 1, 2: 1, 4: 1, 8: 2}.get(world, 2 if world % 2 == 0 else 1)
    Z = int(args.mesh.lower().split("x")[2]) if args.mesh else default_z
    binpath = tmp / "matrix.bin"
    if rank == 0:
        try:
            from baseline import build_reference
            from spcomm3d_b200.utils import binfmt, generate
            tmp.mkdir(parents=True, exist_ok=True)
            for f in (ready, failed):
                if f.exists():
                    f.unlink()
            exe = build_reference.build()
            m = generate.from_spec(args.gen, seed=args.seed)
            binfmt.write_bin(str(binpath), m)
            ready.write_text(str(exe))
        except Exception as e:  # build or generation failed: say why, exit 0
            tmp.mkdir(parents=True, exist_ok=True)
            failed.write_text(str(e)[:300])
    t0 = time.time()
    while not ready.exists() and not failed.exists():
        if time.time() - t0 > 1800:
            if rank == 0:
                _unavailable("timed out preparing the reference build")
            return
        time.sleep(0.2)
    if failed.exists():
        if rank == 0:
            _unavailable(failed.read_text().replace("\n", " "))
        return
    exe = ready.read_text()
    env = dict(os.environ, SP3MPI_RANK=str(rank), SP3MPI_SIZE=str(world), SP3MPI_JOB=f"b{job}")
    t0 = time.time()
    res = subprocess.run([exe, "-k", str(args.k), "-c", str(Z), "-s", str(steps), "-w", str(warmup), "-t", str(BUDGET_S),
                          str(binpath)],
                         capture_output=True, text=True, env=env)
    wall = time.time() - t0
    if rank != 0:
        return
    line = next((l for l in res.stdout.splitlines() if l.startswith("REFDRIVER ")), None)
    if res.returncode != 0 or line is None:
        _unavailable(f"reference driver failed (exit {res.returncode}): {res.stderr[-200:]!r}")
        return
    d = json.loads(line[len("REFDRIVER "):])
    sddmm = min(d["sddmm_sparse_ms"], d["sddmm_sparseNB_ms"])
    value = sddmm + d["spmm_sparse_ms"]
    flops = 2.0 * d["gnnz"] * args.k
    capped = d["steps"] < steps or d["warmup"] < warmup
    out = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world,
        "steps": d["steps"], "warmup": d["warmup"], "ms_per_step": value, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp64", "data": "synthetic", "impl": "reference",
        "timed": "host clock around each call of the reference's distributed kernel, max over ranks",
        "sddmm_ms": sddmm, "spmm_ms": d["spmm_sparse_ms"],
        "sddmm_variants_ms": {"sparse": d["sddmm_sparse_ms"], "sparseNB": d["sddmm_sparseNB_ms"]},
        "sddmm_gflops": flops / sddmm / 1e6, "spmm_gflops": flops / d["spmm_sparse_ms"] / 1e6,
        # operands and results of the reference live in host memory: nothing is copied to or from a device, so
        # the end-to-end time of a step is the step itself
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "CPU code: operands and results are in host memory already"},
        "gpu_launches": 0,
        "hardware": f"host CPU, {world} MPI rank(s) (reference has no GPU path)", "wall_s": round(wall, 1),
        "config": {"model": f"{args.gen} k={args.k} fp64 SDDMM then SpMM", "matrix": args.gen, "nnz": d["gnnz"],
                   "k": args.k, "mesh": d["mesh"], "mpi": "shared-memory MPI subset (baseline/mpi_shim)",
                   "steps_asked": steps, "warmup_asked": warmup, "steps_by_kernel": d["steps_by_kernel"],
                   "steps_cap": (f"wall-clock allowance of {BUDGET_S:g} s per kernel ended the loops early"
                                 if capped else None),
                   "setup_s": round(d["setup_ms"] / 1e3, 1)},
    }
    print(json.dumps(out))
    try:
        binpath.unlink()
    except OSError:
        pass
