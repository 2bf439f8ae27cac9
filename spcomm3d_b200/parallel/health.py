"""Failure detection on the host side.

The reference has none: a missing communicator ends in `exit(EXIT_FAILURE)`
(src/comm.hpp:129-133,160-163) and a lost rank hangs the job.  Here

* `check_consistent` compares a fingerprint of every rank's plan before the
  first launch, so mismatched meshes / matrices / seeds fail with a message
  instead of with wrong pointers;
* `Heartbeat` lets ranks publish their step number in the process group's
  key-value store and lets any rank see, before its next launch, which peers
  have stopped (a rank only ever leaves between steps);
* collectives of the library path end with an error after the process
  group's timeout when a peer never joins, and the device-side waits of the
  fused kernels are bounded and report through a status word
  (csrc/kernels/fused_impl.cuh).

There is no elastic resize: a failed rank ends the job cleanly.
"""
from __future__ import annotations

import hashlib
import time

import numpy as np


class RankFailure(RuntimeError):
    pass


def plan_fingerprint(plan) -> dict:
    h = hashlib.sha256()
    for arr in (plan.row.peer_owned, plan.col.peer_owned):
        h.update(np.ascontiguousarray(arr).tobytes())
    return {"mesh": str(plan.mesh), "dims": (plan.nrows, plan.ncols), "gnnz": plan.gnnz,
            "line_owned": h.hexdigest()}


def check_consistent(plan, groups) -> None:
    """Raises ValueError naming the ranks whose plan disagrees with rank 0 on
    mesh, matrix size, nonzero count, or (within a mesh line) owned counts."""
    import torch.distributed as dist
    mine = plan_fingerprint(plan)
    world = dist.get_world_size()
    allf = [None] * world
    dist.all_gather_object(allf, (plan.rank, mine))
    by_rank = dict(allf)
    ref = by_rank[0]
    bad = [r for r, f in by_rank.items() if any(f[k] != ref[k] for k in ("mesh", "dims", "gnnz"))]
    if sorted(by_rank) != list(range(world)):
        bad.append(-1)
    # ranks of one xy position share the per-line owned counts along Z
    x, y, _ = plan.coords
    for z in range(plan.mesh.Z):
        other = by_rank.get(plan.mesh.rank_of(x, y, z))
        if other is not None and other["line_owned"] != mine["line_owned"]:
            bad.append(plan.mesh.rank_of(x, y, z))
    if bad:
        raise ValueError(f"plans are not consistent across ranks (differing ranks: {sorted(set(bad))}); "
                         "check that every rank uses the same matrix, mesh and seed")


class Heartbeat:
    """Step counters in the default process-group store."""

    def __init__(self, rank: int, world: int, store=None, prefix: str = "sp3hb"):
        if store is None:
            import torch.distributed as dist
            store = dist.distributed_c10d._get_default_store()
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self.beat(0)

    def beat(self, step: int):
        self.store.set(f"{self.prefix}/{self.rank}", f"{step}:{time.time()}")

    def steps(self) -> dict:
        out = {}
        for r in range(self.world):
            try:
                s, t = self.store.get(f"{self.prefix}/{r}").decode().split(":")
                out[r] = (int(s), float(t))
            except Exception:
                out[r] = (-1, 0.0)
        return out

    def require_alive(self, step: int, wait_s: float = 5.0):
        """Waits up to wait_s for every rank to have reached `step`; raises
        RankFailure listing the ranks that have not."""
        deadline = time.time() + wait_s
        while True:
            behind = [r for r, (s, _) in self.steps().items() if s < step]
            if not behind:
                return
            if time.time() > deadline:
                raise RankFailure(f"ranks {behind} did not reach step {step} within {wait_s:.1f} s")
            time.sleep(0.05)
