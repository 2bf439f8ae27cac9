"""Shared pieces of the command-line programs: option parsing in the style of
the reference (`-k k1,k2 -c Z matrix.bin`, miniapp/bench_spmm.cpp:33-103),
process-group start-up and plan construction.

Run single-process (`python -m spcomm3d_b200.cli.bench_sddmm ...`) or under
`torchrun --nproc-per-node N` (one rank per GPU with NCCL, or CPU ranks with
gloo when no GPU is present / `--device cpu`).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

from ..parallel.mesh import Mesh3D, MeshGroups, dims_create
from ..parallel.partition import distribute_from_file
from ..parallel.plan import build_my_plan, build_rank_plan
from ..utils import binfmt, generate

NUM_ITER = 5  # iterations per instance, as miniapp/bench_spmm.cpp:22


def base_parser(prog: str, description: str) -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog=prog, description=description)
    ap.add_argument("matrix", nargs="?", help="matrix in .bin format (or .mtx); omit when --gen is given")
    ap.add_argument("-k", dest="klist", default="32", help="comma separated list of inner dimensions")
    ap.add_argument("-c", "-z", dest="Z", type=int, default=1, help="Z: number of layers the k dimension is split over")
    ap.add_argument("-i", dest="iters", type=int, default=NUM_ITER, help="iterations per instance")
    ap.add_argument("--mesh", default=None, help="XxYxZ; default: balanced X>=Y for the given Z")
    ap.add_argument("--dtype", default=None, choices=["fp32", "fp64"])
    ap.add_argument("--variant", "--variants", dest="variant", default=None,
                    help="comma list of sparse,sparseNRB,fused,fused-atomic,fused-multimem,dense")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--gen", default=None, help="synthetic matrix: uniform:M:N:deg | rmat:scale[:ef] | zipf:M:N[:a[:dmax]] | er:M:N:deg | random:M:N:nnz")
    ap.add_argument("--device", default=None, choices=["cpu", "cuda"])
    ap.add_argument("--policy", default="respect_comm", choices=["respect_comm", "random"])
    ap.add_argument("--json", action="store_true", help="also print one JSON record per instance")
    ap.add_argument("--save-plan", default=None, metavar="PREFIX",
                    help="write every rank's plan to PREFIX.rank<r>.npz after building it")
    ap.add_argument("--load-plan", default=None, metavar="PREFIX",
                    help="read the plans written by --save-plan instead of partitioning the matrix again")
    ap.add_argument("--heartbeat", action="store_true",
                    help="ranks publish their progress in the process-group store; before every instance each rank "
                         "checks that all others have arrived and stops with a message naming the missing ones")
    ap.add_argument("-v", dest="verbose", action="store_true")
    return ap


def klist(text: str):
    return [int(t) for t in text.split(",") if t]


class Runtime:
    def __init__(self, args):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        want_cuda = args.device != "cpu" and torch.cuda.is_available()
        if args.device == "cuda" and not torch.cuda.is_available():
            raise SystemExit("--device cuda but no CUDA device is visible")
        self.device = torch.device("cuda", local) if want_cuda else torch.device("cpu")
        if want_cuda:
            torch.cuda.set_device(self.device)
            from ..utils import affinity
            self.placement = affinity.bind_near_gpu(local, local, int(os.environ.get("LOCAL_WORLD_SIZE", self.world)))
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            # GPU ranks: NCCL for device tensors plus gloo for the host-side collectives of setup (the
            # collective .bin reader exchanges nonzeros and touch masks as host arrays)
            dist.init_process_group("cpu:gloo,cuda:nccl" if want_cuda else "gloo",
                                    **({"device_id": self.device} if want_cuda else {}))
        if args.mesh:
            self.mesh = Mesh3D.parse(args.mesh)
        else:
            if self.world % args.Z:
                raise SystemExit(f"-c {args.Z} does not divide {self.world} ranks")
            self.mesh = Mesh3D(*dims_create(self.world, args.Z))
        if self.mesh.size != self.world:
            raise SystemExit(f"mesh {self.mesh} needs {self.mesh.size} ranks but {self.world} are running")
        self.groups = MeshGroups.create(self.mesh) if self.world > 1 else None
        self.dtype = {"fp32": torch.float32, "fp64": torch.float64, None:
                      (torch.float32 if want_cuda else torch.float64)}[args.dtype]
        self.heartbeat, self._beats = None, 0
        if getattr(args, "heartbeat", False) and self.world > 1:
            from ..parallel.health import Heartbeat
            self.heartbeat = Heartbeat(self.rank, self.world)

    def checkpoint(self, wait_s: float = 60.0):
        """With --heartbeat: publishes that this rank reached the next checkpoint and raises `RankFailure`
        naming the ranks that do not arrive within `wait_s` (a rank only ever leaves between steps, so the
        others learn of it here, on the host, before their next launch)."""
        if self.heartbeat is not None:
            self._beats += 1
            self.heartbeat.beat(self._beats)
            self.heartbeat.require_alive(self._beats, wait_s=wait_s)

    def variants(self, args, default):
        v = args.variant.split(",") if args.variant else list(default)
        if self.device.type != "cuda":
            v = [x for x in v if not x.startswith("fused")]
        if self.dtype != torch.float32:   # the in-switch reduction is built for fp32 only
            v = [x for x in v if x != "fused-multimem"]
        if "fused-multimem" in v and self.mesh.Z != self.world:
            # a multicast binding over part of the job has not been proven on real switches
            self.say(f"# skipping fused-multimem on {self.mesh}: limited to meshes whose Z fiber is the whole job")
            v = [x for x in v if x != "fused-multimem"]
        return v

    def load_plan(self, args):
        """The plan of this rank.  Generated matrices are built identically on
        every rank (no communication); files go through the collective reader.
        --load-plan reads what --save-plan wrote (same mesh and rank count)."""
        from ..parallel.plan import RankPlan
        if getattr(args, "load_plan", None):
            plan = RankPlan.load(f"{args.load_plan}.rank{self.rank}")
            if str(plan.mesh) != str(self.mesh) or plan.rank != self.rank:
                raise SystemExit(f"plan file is for mesh {plan.mesh} rank {plan.rank}, not {self.mesh} rank {self.rank}")
            return plan
        plan = self._build_plan(args)
        if getattr(args, "save_plan", None):
            plan.save(f"{args.save_plan}.rank{self.rank}")
        return plan

    def _build_plan(self, args):
        if args.gen:
            if self.world > 1:   # every rank generates only its own block where the generator allows it
                from ..parallel.plan import build_my_plan_from_spec
                return build_my_plan_from_spec(args.gen, self.mesh, self.groups, seed=args.seed,
                                               policy=args.policy)[1]
            m = generate.from_spec(args.gen, seed=args.seed)
            _, plan = build_my_plan(m, self.mesh, self.rank, seed=args.seed, policy=args.policy)
            return plan
        if not args.matrix:
            raise SystemExit("give a matrix file or --gen")
        path = args.matrix
        if path.endswith(".mtx"):
            m = binfmt.read_mtx(path)
            _, plan = build_my_plan(m, self.mesh, self.rank, seed=args.seed, policy=args.policy)
            return plan
        if self.world == 1:
            m = binfmt.read_bin(path)
            _, plan = build_my_plan(m, self.mesh, 0, seed=args.seed, policy=args.policy)
            return plan
        _, _, gnnz = binfmt.read_bin_header(path)
        block, directory = distribute_from_file(path, self.mesh, self.groups, seed=args.seed, policy=args.policy)
        return build_rank_plan(block, directory, self.groups.coords, gnnz=gnnz)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    def finish(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()

    def say(self, *a):
        if self.rank == 0:
            print(*a)
            sys.stdout.flush()
