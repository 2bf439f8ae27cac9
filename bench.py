"""Headline benchmark: distributed SDDMM + SpMM time per iteration.

    python bench.py --gpus N --steps K --warmup W [--impl reference]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

One step = one distributed SDDMM followed by one distributed SpMM on the same
sparse matrix: R-MAT scale 22, edge factor 16, duplicates removed, k = 128,
fp32, synthetic seeded operands -- the SDDMM and SpMM configurations named for
the 8-GPU comparison.  The total work is fixed as N grows (strong scaling).
`value` is milliseconds per step, device-timed with CUDA events, max over
ranks; lower is better.  Extra keys give the per-kernel times, GFLOP/s
(2*nnz*k per kernel), the communication volume of the plan, the in-kernel phase
stamps of the fused kernels next to the plain local kernels on the same
blocks, and the end-to-end time of the same step through the public API
including the host->device copy of the dense operands from pinned memory and
the device->host read of the two result checksums.

The run checks itself: after every loop all ranks read the status words of
the fused kernels (a wait that ran out or a bad index stops the job without a
number), every rank recomputes a sample of the SDDMM values and SpMM rows it
owns in fp64 from the seeded operand generator (`verified`, `max_rel_err`),
and the two result checksums are summed over all ranks so that they can be
compared across GPU counts and meshes.

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
    ap.add_argument("--no-local", action="store_true", help="skip timing the plain local kernels on each rank's block")
    ap.add_argument("--save-plan", default=None, metavar="PREFIX", help="write every rank's plan to PREFIX.rank<r>.npz")
    ap.add_argument("--load-plan", default=None, metavar="PREFIX", help="read plans written by --save-plan instead of building them")
    return ap.parse_args()


# Fastest mesh per GPU count among those measured on R-MAT-22, k = 128 (fused variant, SDDMM + SpMM per step):
# N=2: 1x2x1 3.64 ms vs 2x1x1 3.79, 1x1x2 4.55; N=4: 2x2x1 2.17 ms vs 4x1x1 2.41, 1x2x2 2.43, 2x1x2 2.67;
# N=8: 2x2x2 1.55 ms vs 4x2x1 2.10, 1x1x8 3.31.
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


METRIC = "SDDMM+SpMM ms/iter (max over ranks)"
UNIT = "ms/iter"
STREAM_A, STREAM_B = 1, 2   # operand streams of models.layer.SddmmSpmmStep
VERIFY_TOL = 1e-4           # sampled results against fp64, relative to the largest reference value


def pick_device(local_rank: int, world: int) -> int:
    """CUDA device of a rank.  With more visible GPUs than ranks the ranks are spread over the node
    (rank r -> device r * visible / world) so that neighbouring ranks do not share a PCIe uplink for their
    host->device copies; SP3_DEVICE_MAP=dense keeps rank r on device r."""
    import torch
    visible = torch.cuda.device_count()
    if os.environ.get("SP3_DEVICE_MAP", "spread") == "spread" and visible > world and visible % world == 0:
        return local_rank * (visible // world)
    return local_rank


def run_ours(args):
    # torchrun pins OMP_NUM_THREADS to 1; matrix generation and plan building (host library, OpenMP) are setup
    # work outside the timed region and may use this rank's share of the cores
    world_env = int(os.environ.get("WORLD_SIZE", 1))
    if os.environ.get("OMP_NUM_THREADS") == "1" and world_env > 1:
        os.environ["OMP_NUM_THREADS"] = str(max(1, min(16, (os.cpu_count() or 1) // world_env)))
    import numpy as np
    import torch
    import torch.distributed as dist
    from spcomm3d_b200.models import verify
    from spcomm3d_b200.models.layer import SddmmSpmmStep
    from spcomm3d_b200.ops import cuda_ops
    from spcomm3d_b200.parallel import health
    from spcomm3d_b200.parallel.mesh import Mesh3D, MeshGroups
    from spcomm3d_b200.parallel.plan import RankPlan, build_my_plan, build_my_plan_from_spec
    from spcomm3d_b200.utils import affinity, generate, native

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    dev_index = pick_device(local_rank, world)
    torch.cuda.set_device(dev_index)
    device = torch.device("cuda", dev_index)
    # pinned staging buffers and the threads that fill them: on the NUMA node of this rank's GPU
    placement = affinity.bind_near_gpu(dev_index, local_rank, world)
    native.cuda()
    groups = None
    if world > 1:
        # NCCL moves device tensors; gloo serves the host-side collectives of setup (plan fingerprints)
        dist.init_process_group("cpu:gloo,cuda:nccl", device_id=device)
    mesh = Mesh3D.parse(args.mesh) if args.mesh else Mesh3D(*default_mesh(world))
    if mesh.size != world:
        raise SystemExit(f"mesh {mesh} does not match {world} ranks")
    if world > 1:
        groups = MeshGroups.create(mesh)
    variant = args.variant or ("fused" if world > 1 else "sparseNRB")
    if variant == "fused-multimem" and mesh.Z != world:
        raise SystemExit("fused-multimem is limited to meshes whose Z fiber is the whole job (1x1xZ)")

    # Setup: every rank builds its own block where the generator can be restricted to one (uniform, zipf, er);
    # R-MAT removes duplicates globally, so every rank generates it whole (1.6 s at scale 22).
    t0 = time.time()
    m = None
    if args.load_plan:
        plan = RankPlan.load(f"{args.load_plan}.rank{rank}")
    elif world > 1:
        _, plan, m = build_my_plan_from_spec(args.gen, mesh, groups, seed=args.seed)
    else:
        m = generate.from_spec(args.gen, seed=args.seed)
        _, plan = build_my_plan(m, mesh, rank, seed=args.seed)
    if args.save_plan:
        plan.save(f"{args.save_plan}.rank{rank}")
    gnnz = plan.gnnz
    setup_s = time.time() - t0
    gen_s = None
    if m is None:   # rows of the whole matrix for the sampled check are generated on demand
        if generate._spec_rowptr(args.gen, args.seed) is not None:
            def m(gids, spec=args.gen, seed=args.seed):
                return generate.rows_from_spec(spec, seed, gids)
        else:
            m = generate.from_spec(args.gen, seed=args.seed)
    if world > 1:
        health.check_consistent(plan, groups)   # same matrix, mesh and seed on every rank, before any launch
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

    def reduce(values, op):
        t = torch.tensor(list(values), dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=op)
        return t.tolist()

    def maxr(x):
        return reduce([x], dist.ReduceOp.MAX)[0]

    def agree_healthy(where: str):
        """Reads the status words of the fused kernels on every rank; one failing rank stops the whole job
        with its message (no number is printed for a run whose kernels did not complete)."""
        msg = ""
        try:
            step.check()
        except Exception as e:
            msg = f"rank {rank} {where}: {e}"
        if maxr(1.0 if msg else 0.0) > 0:
            if msg:
                print(msg, file=sys.stderr)
            try:
                step.close()
            except Exception:
                pass
            raise SystemExit(f"bench aborted: a fused kernel reported a failure {where}")

    # ---- kernel-path timing: operands resident on the device --------------
    for _ in range(args.warmup):
        step.run_device()
    barrier()
    agree_healthy("after warm-up")
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    sampler = ClockSampler(dev_index)   # NVML start-up happens here, before the barrier that opens the timed region
    with sampler as clocks:
        barrier()                       # every rank enters the timed region together
        launches0 = cuda_ops.LAUNCHES
        ev[0].record()
        for i in range(args.steps):
            step.sddmm.run_async()
            ev[2 * i + 1].record()
            step.spmm.run_async()
            ev[2 * i + 2].record()
        barrier()
    launches = cuda_ops.LAUNCHES - launches0
    agree_healthy("in the timed loop")
    total_ms = maxr(ev[0].elapsed_time(ev[-1]))
    sddmm_ms = maxr(sum(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(args.steps)) / args.steps)
    spmm_ms = maxr(sum(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(args.steps)) / args.steps)
    ms_per_step = total_ms / args.steps

    # in-kernel phase stamps of the last fused launches and the plain local kernels on the same blocks
    phases = None
    ph = step.phase_ms()
    if ph is not None:
        flat = [ph[op][key] for op in ("sddmm", "spmm") for key in ("pull", "main", "total")]
        flat = reduce(flat, dist.ReduceOp.MAX)
        phases = {op: {key: round(flat[3 * i + j], 4) for j, key in enumerate(("pull", "main", "total"))}
                  for i, op in enumerate(("sddmm", "spmm"))}
    local_ms = None
    if world > 1 and not args.no_local:
        lsd, lsp = step.local_kernel_ms()
        lsd, lsp = reduce([lsd, lsp], dist.ReduceOp.MAX)
        local_ms = {"sddmm": round(lsd, 4), "spmm": round(lsp, 4),
                    "note": "plain local kernels on each rank's block with all dense rows resident, max over ranks"}

    # ---- correctness: a sample of every rank's results against fp64, and global checksums ----
    c, y = step.run_device()
    agree_healthy("in the verification step")
    err_sd = verify.sample_sddmm_error(plan, c, args.k, args.seed, STREAM_A, STREAM_B,
                                       positions=step.sddmm.owned_positions())
    err_sp = verify.sample_spmm_error(plan, m, y, args.k, args.seed, STREAM_B)
    del m
    err_sd, err_sp = reduce([err_sd, err_sp], dist.ReduceOp.MAX)
    sums = reduce([float(cuda_ops.checksum(c)), float(cuda_ops.checksum(y.reshape(-1)))], dist.ReduceOp.SUM)
    verified = bool(err_sd < VERIFY_TOL and err_sp < VERIFY_TOL and np.isfinite(sums).all())

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
        agree_healthy("in the end-to-end loop")
        e2e_ms = maxr(a.elapsed_time(b)) / args.steps
        gsum = reduce(res, dist.ReduceOp.SUM)
        e2e = {"value": e2e_ms, "unit": UNIT,
               "note": "SDDMM+SpMM incl. H2D of A and B from pinned memory and D2H of the two result checksums, every step",
               "h2d_bytes_per_step": step.h2d_bytes, "d2h_bytes_per_step": step.d2h_bytes,
               "global_checksums": gsum,
               "checksums_match_device_path": bool(np.allclose(gsum, sums, rtol=1e-6, atol=1e-3))}

    vol_t = reduce(step.comm_volume_bytes(), dist.ReduceOp.SUM)
    flops = 2.0 * gnnz * args.k
    out = {
        "metric": METRIC, "value": ms_per_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "ours",
        "timed": "CUDA events on the launching stream, max over ranks",
        "sddmm_ms": sddmm_ms, "spmm_ms": spmm_ms,
        "sddmm_gflops": flops / sddmm_ms / 1e6, "spmm_gflops": flops / spmm_ms / 1e6,
        "comm_bytes_per_step": {"sddmm_expand": vol_t[0], "sddmm_zreduce": vol_t[1],
                                "spmm_expand": vol_t[2], "spmm_reduce": vol_t[3]},
        "verified": verified, "max_rel_err": {"sddmm": err_sd, "spmm": err_sp},
        "global_checksums": {"sddmm": sums[0], "spmm": sums[1]},
        "fused_phase_ms": phases, "local_kernel_ms": local_ms,
        "gpu_launches": launches, "clocks": clocks.summary(), "e2e": e2e,
        "config": {"model": f"{args.gen} k={args.k} fp32 SDDMM then SpMM", "matrix": args.gen, "nnz": gnnz,
                   "k": args.k, "mesh": str(mesh), "variant": variant, "precision": "tf32 panels + fp32" if args.panels else "fp32", "global_batch": None, "seq_len": None,
                   "parallelism": f"mesh{mesh}", "l2": "operands larger than L2 at every N; no flush",
                   "device_of_rank0": dev_index, "numa_of_rank0": placement, "setup_s": round(setup_s, 1)},
    }
    if not verified:
        print(f"verification FAILED: max rel err sddmm {err_sd:.3e}, spmm {err_sp:.3e}", file=sys.stderr)
    if rank == 0:
        print(json.dumps(out))
    step.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not verified:
        raise SystemExit(3)


def run_reference(args):
    from baseline import reference_arm
    reference_arm.run(args, METRIC, UNIT)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
