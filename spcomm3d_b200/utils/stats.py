"""Communication / timing statistics in the reference's line format, JSON
records and roofline arithmetic.

Line layout (whitespace separated), one line per (iteration, phase), as
printed by src/comm_stats.cpp:33-36,53:

  <mtxName> <algName> <P> <k> <Z>  <avgSendMsgs> <avgSendVol> <avgRecvMsgs> <avgRecvVol>
  <maxSendMsgs> <maxSendVol> <maxRecvMsgs> <maxRecvVol>  <comm1> <comm2> <commcpy> <comp> <total>

`algName` contains spaces ("sparse sddmm PRE").  Volumes are element counts
(rows x k/Z), messages are neighbour counts (src/comm_stats.cpp:62-65); the
times are those of the rank with the largest total (src/comm_stats.cpp:42-57).
The reference truncates times to integer milliseconds (src/basic.hpp:20-22);
here they are printed with three decimals, which every whitespace/float parser
of the original layout accepts.
"""
from __future__ import annotations

import json

import torch

PHASES = ("PRE", "POST")
TIME_KEYS = ("comm1", "comm2", "commcpy", "comp", "total")


def _device_for(group_backend_device):
    return group_backend_device


def aggregate(op, phase: str, groups=None):
    """Sums / maxima of this op's per-rank message and volume counts over all
    ranks, plus the phase times of the slowest rank."""
    import torch.distributed as dist
    (smsg, svol), (rmsg, rvol) = op.comm_stats()[phase]
    mine = torch.tensor([smsg, svol, rmsg, rvol], dtype=torch.float64)
    times = torch.tensor([op.last_times.get(k, 0.0) for k in TIME_KEYS], dtype=torch.float64)
    world = op.mesh.size
    if groups is not None and world > 1:
        dev = op.device if op.device.type == "cuda" else torch.device("cpu")
        tot, mx = mine.to(dev).clone(), mine.to(dev).clone()
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        all_t = torch.empty(world, len(TIME_KEYS), dtype=torch.float64, device=dev)
        dist.all_gather_into_tensor(all_t.view(-1), times.to(dev))
        slow = int(torch.argmax(all_t[:, TIME_KEYS.index("total")]))
        tot, mx, times = tot.cpu(), mx.cpu(), all_t[slow].cpu()
    else:
        tot, mx, slow = mine, mine, 0
    return {"avg": (tot / world).tolist(), "max": mx.tolist(), "times": times.tolist(), "slowest_rank": slow}


def format_line(mtx_name: str, alg_name: str, P: int, k: int, Z: int, agg: dict) -> str:
    a, m, t = agg["avg"], agg["max"], agg["times"]
    return (f"{mtx_name} {alg_name} {P} {k} {Z} {a[0]:.2f} {a[1]:.2f} {a[2]:.2f} {a[3]:.2f} "
            f"{int(m[0])} {int(m[1])} {int(m[2])} {int(m[3])} "
            + " ".join(f"{x:.3f}" for x in t))


def parse_line(line: str) -> dict:
    """Inverse of format_line; also parses lines printed by the reference."""
    tok = line.split()
    # algName is everything between the matrix name and the first of 16 trailing numeric fields
    tail = tok[-16:]
    return {"mtx": tok[0], "alg": " ".join(tok[1:-16]), "P": int(tail[0]), "k": int(tail[1]), "Z": int(tail[2]),
            "avg": [float(x) for x in tail[3:7]], "max": [float(x) for x in tail[7:11]],
            "times": dict(zip(TIME_KEYS, (float(x) for x in tail[11:16])))}


def report_iteration(op, groups=None, rank: int = 0, out=print):
    """Prints the PRE and POST lines of the op's last run (rank 0 prints) and
    returns the two aggregates."""
    aggs = {}
    for phase in PHASES:
        agg = aggregate(op, phase, groups)
        aggs[phase] = agg
        if rank == 0:
            out(format_line(op.plan.name, op.alg_name(phase), op.mesh.size, op.k, op.mesh.Z, agg))
    return aggs


def measured_peaks(path: str | None = None) -> dict:
    """{"hbm_gbs", "nvlink_gbs", "source"}: denominators of the rooflines.  Defaults: 6549.8 GB/s for a
    device-memory copy and 770 GB/s per direction for a peer copy over NVLink (both measured on B200 boxes).
    A JSON file with a key `hbm_gbs` overrides the first; it is looked for at `path`, else at the path in the
    environment variable SP3_PEAKS_FILE; SP3_HBM_GBS / SP3_NVLINK_GBS override single figures."""
    import os
    out = {"hbm_gbs": 6549.8, "nvlink_gbs": 770.0, "source": "built-in"}
    path = path or os.environ.get("SP3_PEAKS_FILE")
    if path:
        try:
            with open(path) as f:
                d = json.load(f)
            if float(d.get("hbm_gbs", 0)) > 0:
                out["hbm_gbs"], out["source"] = float(d["hbm_gbs"]), os.path.basename(path)
        except (OSError, ValueError):
            pass
    for key, env in (("hbm_gbs", "SP3_HBM_GBS"), ("nvlink_gbs", "SP3_NVLINK_GBS")):
        if os.environ.get(env):
            out[key], out["source"] = float(os.environ[env]), "environment"
    return out


def roofline(flops: float, nvlink_bytes_per_rank: float, hbm_bytes_per_rank: float, ms: float,
             peak_tflops: float = 70.0, nvlink_gbs: float = 770.0, hbm_gbs: float = 6549.8) -> dict:
    """Roofline of a fused op: the slower of its FLOPs at peak and the bytes it must move over NVLink at link
    bandwidth (`floor_ms`, `fraction` = floor / measured time, `bound`).  `peak_tflops` is the fp32 FMA peak
    that applies to these kernels (not the tensor-core peak).

    A second, informative figure: `gather_model_ms` = the dense rows the local kernel fetches (one row per
    nonzero, no reuse) at the device-memory copy rate, with `gather_model_fraction`.  It is a model of the
    local gather without cache reuse, not a bound: a kernel whose rows are served by the L2 beats it."""
    t_flop = flops / (peak_tflops * 1e12) * 1e3
    t_link = nvlink_bytes_per_rank / (nvlink_gbs * 1e9) * 1e3
    t_hbm = hbm_bytes_per_rank / (hbm_gbs * 1e9) * 1e3
    floor = max(t_flop, t_link)
    return {"floor_ms": floor, "flop_ms": t_flop, "nvlink_ms": t_link,
            "fraction": floor / ms if ms > 0 else 0.0,
            "bound": "flops" if t_flop >= t_link else "nvlink",
            "gather_model_ms": t_hbm, "gather_model_fraction": t_hbm / ms if ms > 0 else 0.0}


def json_record(op, kernel: str, ms: float, extra: dict | None = None) -> str:
    rec = {"kernel": kernel, "matrix": op.plan.name, "mesh": str(op.mesh), "k": op.k, "variant": op.variant,
           "ms_per_iter": ms, "gflops": op.flops() / ms / 1e6 if ms > 0 else None,
           "comm": {ph: {"send_msgs": s[0], "send_elems": s[1], "recv_msgs": r[0], "recv_elems": r[1]}
                    for ph, (s, r) in op.comm_stats().items()}}
    if extra:
        rec.update(extra)
    return json.dumps(rec)
