"""Headline benchmark: distributed SDDMM + SpMM time per iteration.

    python bench.py --gpus N --steps K --warmup W [--impl reference]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

One step = one distributed SDDMM followed by one distributed SpMM on the same
sparse matrix: R-MAT scale 22, edge factor 16, duplicates removed, k = 128,
fp32, synthetic seeded operands -- the SDDMM and SpMM configurations named for
the 8-GPU comparison.  The total work is fixed as N grows (strong scaling).
`value` is milliseconds per step, device-timed with CUDA events, max over
ranks; lower is better.  Extra keys give the per-kernel times, GFLOP/s
(2*nnz*k per kernel), the communication volume of the plan and the end-to-end
time of the same step through the public API including the host->device copy
of the dense operands from pinned memory and the device->host read of the two
result checksums.

Operands are larger than the L2 cache at every N (>= 0.5 GB per rank), so no
L2 flush is interleaved; `config.l2` states this.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gen", default="rmat:22:16", help="matrix spec (utils.generate.from_spec)")
    ap.add_argument("--k", type=int, default=128)
    ap.add_argument("--mesh", default=None, help="XxYxZ (default: the fastest measured mesh for N = 2, 4, 8)")
    ap.add_argument("--variant", default=None,
                    choices=[None, "fused", "fused-atomic", "fused-multimem", "sparse", "sparseNRB", "dense"])
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--panels", action="store_true",
                    help="SDDMM and SpMM: dense 128x64 panels on the tcgen05 tensor cores (TF32), rest on the gather kernels")
    ap.add_argument("--min-col-nnz", type=int, default=3)
    return ap.parse_args()


# Fastest mesh per GPU count among those measured on this matrix (fused variant, SDDMM + SpMM):
# N=2: 1x2x1 1.07 ms vs 2x1x1 1.17, 1x1x2 1.23 (R-MAT-20); N=4: 2x2x1 2.49 ms vs 1x2x2 2.70, 2x1x2 2.94;
# N=8: 2x2x2 1.99 ms vs 4x2x1 2.05 (R-MAT-22).
MEASURED_MESH = {1: (1, 1, 1), 2: (1, 2, 1), 4: (2, 2, 1), 8: (2, 2, 2)}


def default_mesh(world: int):
    if world in MEASURED_MESH:
        return MEASURED_MESH[world]
    from spcomm3d_b200.parallel.mesh import dims_create
    return dims_create(world, 2 if world % 2 == 0 else 1)


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read
    only) while the timed region runs."""

    def __init__(self, index: int, period=0.004):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.period = period

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()
        return False

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def run_ours(args):
    # torchrun pins OMP_NUM_THREADS to 1; matrix generation and plan building (host library, OpenMP) are setup
    # work outside the timed region and may use this rank's share of the cores
    world_env = int(os.environ.get("WORLD_SIZE", 1))
    if os.environ.get("OMP_NUM_THREADS") == "1" and world_env > 1:
        os.environ["OMP_NUM_THREADS"] = str(max(1, min(16, (os.cpu_count() or 1) // world_env)))
    import torch
    import torch.distributed as dist
    from spcomm3d_b200.models.layer import SddmmSpmmStep
    from spcomm3d_b200.ops import cuda_ops
    from spcomm3d_b200.parallel.mesh import Mesh3D, MeshGroups, dims_create
    from spcomm3d_b200.parallel.plan import build_my_plan
    from spcomm3d_b200.utils import generate, native

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    native.cuda()
    groups = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    mesh = Mesh3D.parse(args.mesh) if args.mesh else Mesh3D(*default_mesh(world))
    if mesh.size != world:
        raise SystemExit(f"mesh {mesh} does not match {world} ranks")
    if world > 1:
        groups = MeshGroups.create(mesh)
    variant = args.variant or ("fused" if world > 1 else "sparseNRB")

    t0 = time.time()
    m = generate.from_spec(args.gen, seed=args.seed)
    directory, plan = build_my_plan(m, mesh, rank, seed=args.seed)
    gnnz = m.nnz
    del m
    setup_s = time.time() - t0
    kw = {"panels": True, "min_col_nnz": args.min_col_nnz} if args.panels else {}
    step = SddmmSpmmStep(plan, groups, args.k, torch.float32, device, variant, seed=args.seed, **kw)
    if args.panels and step.sddmm._panels is not None and rank == 0:
        pn = step.sddmm._panels
        print(f"# panels: {pn.npanels} tiles hold {pn.n_panel_nnz} of {pn.nnz} nonzeros", file=sys.stderr)
    step.fill_device_operands()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def maxr(x):
        t = torch.tensor([x], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    # ---- kernel-path timing: operands resident on the device --------------
    for _ in range(args.warmup):
        step.run_device()
    barrier()
    launches0 = cuda_ops.LAUNCHES
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3 * args.steps + 1)]
    with ClockSampler(local_rank) as clocks:
        ev[0].record()
        for i in range(args.steps):
            step.sddmm.run_async()
            ev[3 * i + 1].record()
            step.spmm.run_async()
            ev[3 * i + 2].record()
            ev[3 * i + 3].record()
        barrier()
    launches = cuda_ops.LAUNCHES - launches0
    total_ms = maxr(ev[0].elapsed_time(ev[-1]))
    sddmm_ms = maxr(sum(ev[3 * i].elapsed_time(ev[3 * i + 1]) for i in range(args.steps)) / args.steps)
    spmm_ms = maxr(sum(ev[3 * i + 1].elapsed_time(ev[3 * i + 2]) for i in range(args.steps)) / args.steps)
    ms_per_step = total_ms / args.steps

    # ---- end to end through the public API ---------------------------------
    e2e = None
    if not args.no_e2e:
        step.make_host_operands()
        for _ in range(max(1, min(args.warmup, 2))):
            step.run_e2e()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            res = step.run_e2e()
        b.record()
        barrier()
        e2e_ms = maxr(a.elapsed_time(b)) / args.steps
        e2e = {"value": e2e_ms, "unit": "ms/iter (SDDMM+SpMM, incl. H2D of A and B from pinned memory + D2H of the two checksums)",
               "h2d_bytes_per_step": step.h2d_bytes, "d2h_bytes_per_step": step.d2h_bytes,
               "checksums": [float(x) for x in res]}

    vol = step.comm_volume_bytes()
    vol_t = torch.tensor(vol, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(vol_t)
    flops = 2.0 * gnnz * args.k
    out = {
        "metric": "SDDMM+SpMM ms/iter (device-timed, max over ranks)",
        "value": ms_per_step, "unit": "ms/iter", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic", "impl": "ours",
        "sddmm_ms": sddmm_ms, "spmm_ms": spmm_ms,
        "sddmm_gflops": flops / sddmm_ms / 1e6, "spmm_gflops": flops / spmm_ms / 1e6,
        "comm_bytes_per_step": {"sddmm_expand": vol_t[0].item(), "sddmm_zreduce": vol_t[1].item(),
                                "spmm_expand": vol_t[2].item(), "spmm_reduce": vol_t[3].item()},
        "gpu_launches": launches, "clocks": clocks.summary(), "e2e": e2e,
        "config": {"model": f"{args.gen} k={args.k} fp32 SDDMM then SpMM", "matrix": args.gen, "nnz": gnnz,
                   "k": args.k, "mesh": str(mesh), "variant": variant, "precision": "tf32 panels + fp32" if args.panels else "fp32", "global_batch": None, "seq_len": None,
                   "parallelism": f"mesh{mesh}", "l2": "operands larger than L2 at every N; no flush",
                   "setup_s": round(setup_s, 1)},
    }
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    from baseline import reference_arm
    reference_arm.run(args)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
