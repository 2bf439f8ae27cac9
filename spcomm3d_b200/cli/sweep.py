"""sweep: SDDMM and SpMM over several meshes / variants / k on the running ranks.

    torchrun --nproc-per-node N -m spcomm3d_b200.cli.sweep --gen rmat:22:16 -k 128 \
        --meshes 2x2x2,4x2x1,1x1x8 --variants fused,sparseNRB,dense

Prints one JSON line per (mesh, variant, k, kernel): device-timed ms/iter (max
over ranks), GFLOP/s, the plan's communication volume (max and sum over ranks,
bytes actually needed = the sparsity-aware minimum), and for the fused
variant the in-kernel pull time and the achieved fraction of the roofline
max(FLOPs / peak, bytes needed over NVLink / link bandwidth); the no-reuse
gather model (one dense row per nonzero at the device-memory copy rate) is
printed beside it for orientation.  This is the programme that fills the
comparison grid of meshes the reference runs by hand with different `-c`
values (miniapp/bench_spmm.cpp:137-143).
"""
from __future__ import annotations

import json
import sys

import torch

from ..models.dist_ops import DistSDDMM, DistSpMM
from ..parallel.mesh import Mesh3D, MeshGroups
from ..parallel.plan import build_my_plan
from ..utils import generate, stats
from .common import Runtime, base_parser, klist

_PEAKS = stats.measured_peaks()   # roofline denominators: measured copy bandwidth, measured NVLink peer copy
NVLINK_GBS, HBM_GBS = _PEAKS["nvlink_gbs"], _PEAKS["hbm_gbs"]


def main(argv=None):
    ap = base_parser("sweep", __doc__.split("\n")[0])
    ap.add_argument("--meshes", default=None, help="comma list of XxYxZ (default: the mesh given by -c)")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--chain", action="store_true",
                    help="also time the attention-style chain Y = (S o (A B^T)) X (SDDMM scores as SpMM values)")
    args = ap.parse_args(argv)
    rt = Runtime(args)
    import torch.distributed as dist
    from ..parallel.plan import build_my_plan_from_spec
    m = None
    if not args.gen:
        from ..utils import binfmt
        m = binfmt.read_mtx(args.matrix) if args.matrix.endswith(".mtx") else binfmt.read_bin(args.matrix)
    elif rt.world == 1 or generate._spec_rowptr(args.gen, args.seed) is None:
        m = generate.from_spec(args.gen, seed=args.seed)   # generators that cannot be restricted to a block
    meshes = [Mesh3D.parse(t) for t in args.meshes.split(",")] if args.meshes else [rt.mesh]
    for mesh in meshes:
        if mesh.size != rt.world:
            rt.say(f"# skipping mesh {mesh}: needs {mesh.size} ranks")
            continue
        groups = MeshGroups.create(mesh) if rt.world > 1 else None
        if m is not None:
            _, plan = build_my_plan(m, mesh, rt.rank, seed=args.seed, policy=args.policy)
        else:   # every rank generates its own block only
            _, plan, _ = build_my_plan_from_spec(args.gen, mesh, groups, seed=args.seed, policy=args.policy)
        for k in klist(args.klist):
            for variant in rt.variants(args, ("fused", "sparseNRB", "dense")):
                for cls in (DistSDDMM, DistSpMM):
                    try:
                        op = cls(plan, groups, k, rt.dtype, rt.device, variant)
                    except ValueError as e:
                        rt.say(f"# skipping {variant} {cls.kernel} on {mesh} k={k}: {e}")
                        continue
                    for name, side, stream in (("A_owned", plan.row, 1), ("B_owned", plan.col, 2),
                                               ("X_owned", plan.col, 2)):
                        if hasattr(op, name):
                            op.fill_owned(getattr(op, name), side.owned_gids, seed=args.seed, stream=stream)
                    for _ in range(args.warmup):
                        op.run_async()
                    rt.barrier()
                    cuda = rt.device.type == "cuda"
                    if cuda:
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record()
                    else:
                        import time
                        t0 = time.perf_counter()
                    for _ in range(args.steps):
                        op.run_async()
                    if cuda:
                        b.record()
                        rt.barrier()
                        ms = a.elapsed_time(b) / args.steps
                    else:
                        rt.barrier()
                        ms = (time.perf_counter() - t0) * 1e3 / args.steps
                    es = 4 if rt.dtype == torch.float32 else 8
                    cs = op.comm_stats()
                    recv_bytes = (cs["PRE"][1][1] + (cs["POST"][1][1] if cls is DistSpMM else 0)) * es
                    if cls is DistSDDMM and mesh.Z > 1:
                        recv_bytes += (plan.nnz - cs["POST"][1][1]) * es  # partial values from the fiber
                    gather_bytes = plan.nnz * op.k_loc * es  # dense rows fetched by the local kernel
                    vec = torch.tensor([ms, recv_bytes, recv_bytes, 0.0, 0.0], dtype=torch.float64, device=rt.device)
                    if op.variant == "fused":
                        ph = op._fused.phase_ms()
                        vec[3], vec[4] = ph["pull"], ph["main"]
                    if rt.world > 1:
                        mx = vec.clone()
                        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
                        sm = vec.clone()
                        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
                    else:
                        mx = sm = vec
                    ms_max = float(mx[0])
                    roof = stats.roofline(op.flops() / mesh.size, float(mx[1]), gather_bytes, ms_max,
                                          nvlink_gbs=NVLINK_GBS, hbm_gbs=HBM_GBS)
                    rec = {"kernel": cls.kernel, "mesh": str(mesh), "variant": variant, "path": op.variant, "k": k,
                           "matrix": plan.name,
                           "ms": round(ms_max, 4), "gflops": round(op.flops() / ms_max / 1e6, 1),
                           "comm_bytes_max_rank": float(mx[1]), "comm_bytes_total": float(sm[2]),
                           "roofline": {kk: (round(v, 4) if isinstance(v, float) else v) for kk, v in roof.items()}}
                    if op.variant == "fused":
                        rec["pull_ms"] = round(float(mx[3]), 4)
                        rec["main_ms"] = round(float(mx[4]), 4)
                    rt.say(json.dumps(rec))
                    op.close()   # collective: status check, multicast binding dropped by all ranks together
                    del op
                if args.chain and variant in ("fused", "sparseNRB", "sparse"):
                    from ..models.layer import GatLayer
                    layer = GatLayer(plan, groups, k, rt.dtype, rt.device, variant)
                    layer.sddmm.fill_owned(layer.sddmm.A_owned, plan.row.owned_gids, seed=args.seed, stream=1)
                    layer.sddmm.fill_owned(layer.sddmm.B_owned, plan.col.owned_gids, seed=args.seed, stream=2)
                    layer.spmm.fill_owned(layer.spmm.X_owned, plan.col.owned_gids, seed=args.seed, stream=2)
                    for op_ in (layer.sddmm, layer.spmm):
                        op_.timer.enabled = False
                    for _ in range(args.warmup):
                        layer.run()
                    rt.barrier()
                    if rt.device.type == "cuda":
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record()
                    else:
                        import time
                        t0 = time.perf_counter()
                    for _ in range(args.steps):
                        layer.run()
                    if rt.device.type == "cuda":
                        b.record()
                        rt.barrier()
                        ms = a.elapsed_time(b) / args.steps
                    else:
                        rt.barrier()
                        ms = (time.perf_counter() - t0) * 1e3 / args.steps
                    t = torch.tensor([ms], dtype=torch.float64, device=rt.device)
                    if rt.world > 1:
                        dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    rt.say(json.dumps({"kernel": "sddmm->spmm chain", "mesh": str(mesh), "variant": variant, "k": k,
                                       "matrix": plan.name, "ms": round(float(t), 4),
                                       "gflops": round(2 * layer.sddmm.flops() / float(t) / 1e6, 1)}))
                    layer.sddmm.close()
                    layer.spmm.close()
                    del layer
    rt.finish()


if __name__ == "__main__":
    main(sys.argv[1:])
