"""Stats line format, CLI programs under torchrun (gloo), host-side failure detection."""
import datetime
import os
import subprocess
import sys

import pytest
import torch

from dist_utils import ROOT, free_port, run_ranks
from spcomm3d_b200.utils import binfmt, generate, stats

ENV = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1")


def test_stats_line_roundtrip_and_reference_layout():
    agg = {"avg": [1.5, 2048.0, 1.5, 2000.25], "max": [2, 4096, 2, 4000], "times": [1.0, 2.0, 0.5, 3.0, 6.0]}
    line = stats.format_line("web", "sparse sddmm PRE", 8, 128, 2, agg)
    assert len(line.split()) == 2 + 2 + 16  # name, 3-word alg, 16 numeric fields
    p = stats.parse_line(line)
    assert p["alg"] == "sparse sddmm PRE" and p["P"] == 8 and p["k"] == 128 and p["Z"] == 2
    assert p["max"] == [2, 4096, 2, 4000] and p["times"]["total"] == 6.0
    # a line as the reference prints it (integer milliseconds)
    ref = "web sparseNB sddmm POST 8 128 2 1.00 10.00 1.00 5.00 1 10 1 5 3 1 0 7 11"
    q = stats.parse_line(ref)
    assert q["alg"] == "sparseNB sddmm POST" and q["times"]["comp"] == 7.0


def test_roofline_picks_the_slowest_resource():
    r = stats.roofline(flops=2e9, nvlink_bytes_per_rank=0.5e9, hbm_bytes_per_rank=1e9, ms=1.0)
    assert r["bound"] == "nvlink" and abs(r["nvlink_ms"] - 0.5e9 / 770e9 * 1e3) < 1e-9 and 0 < r["fraction"] < 1
    # the no-reuse gather model is reported beside the roofline, never as its floor
    big = stats.roofline(flops=2e9, nvlink_bytes_per_rank=0.5e9, hbm_bytes_per_rank=1e12, ms=1.0)
    assert big["floor_ms"] == r["floor_ms"] and big["gather_model_ms"] > big["floor_ms"]
    r = stats.roofline(flops=2e15, nvlink_bytes_per_rank=0.0, hbm_bytes_per_rank=0.0, ms=100.0)
    assert r["bound"] == "flops"


def _torchrun(n, module, *args):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), "-m", module, *args]
    return subprocess.run(cmd, capture_output=True, text=True, env=ENV, timeout=300, cwd=ROOT)


def test_bench_cli_under_torchrun_prints_parsable_lines(tmp_path):
    m = generate.fixed_degree(400, 300, 5, seed=1)
    path = str(tmp_path / "web.bin")
    binfmt.write_bin(path, m)
    out = _torchrun(4, "spcomm3d_b200.cli.bench_sddmm", "-k", "8,16", "-c", "2", "-i", "2", "--device", "cpu", path)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("web ")]
    # 2 k values x 3 CPU variants x 2 iterations x 2 phases
    assert len(lines) == 2 * 3 * 2 * 2
    algs = {stats.parse_line(l)["alg"] for l in lines}
    assert algs == {f"{v} sddmm {p}" for v in ("sparse", "sparseNRB", "dense") for p in ("PRE", "POST")}
    pre = [stats.parse_line(l) for l in lines if "sparseNRB sddmm PRE" in l and " 16 2 " in l][0]
    assert pre["P"] == 4 and pre["avg"][1] == pre["avg"][3]  # everything sent is received
    dense = [stats.parse_line(l) for l in lines if "dense sddmm PRE" in l and " 16 2 " in l][0]
    assert dense["avg"][3] >= pre["avg"][3]
    # --heartbeat: every rank publishes its progress and checks the others before each instance
    out = _torchrun(2, "spcomm3d_b200.cli.bench_spmm", "-k", "8", "-c", "1", "-i", "1", "--device", "cpu", "--heartbeat",
                    path)
    assert out.returncode == 0, out.stderr[-2000:]
    assert sum(l.startswith("web ") for l in out.stdout.splitlines()) == 3 * 2


def test_sweep_cli_reports_every_mesh_and_variant():
    import json
    out = _torchrun(2, "spcomm3d_b200.cli.sweep", "--gen", "zipf:900:1200:1.5:200", "-k", "16", "--meshes",
                    "2x1x1,1x2x1,1x1x2,2x2x1", "--variants", "sparseNRB,dense,fused", "--steps", "2", "--warmup", "1",
                    "--device", "cpu")
    assert out.returncode == 0, out.stderr[-2000:]
    recs = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    # three 2-rank meshes (2x2x1 is skipped) x two CPU variants (fused needs GPUs) x two kernels
    assert len(recs) == 3 * 2 * 2
    assert {r["mesh"] for r in recs} == {"2x1x1", "1x2x1", "1x1x2"}
    by = {(r["mesh"], r["variant"], r["kernel"]): r for r in recs}
    for mesh in ("2x1x1", "1x2x1"):
        for kern in ("sddmm", "spmm"):
            assert by[(mesh, "sparseNRB", kern)]["comm_bytes_total"] <= by[(mesh, "dense", kern)]["comm_bytes_total"]
    for r in recs:
        assert r["ms"] > 0 and r["roofline"]["floor_ms"] >= 0 and r["roofline"]["bound"] in ("nvlink", "flops")


def test_checksum_tools_agree(tmp_path):
    from spcomm3d_b200.cli import num_check_seq
    m = generate.fixed_degree(300, 300, 4, seed=2)
    mtx, binp = str(tmp_path / "c.mtx"), str(tmp_path / "c.bin")
    binfmt.write_mtx(mtx, m)
    binfmt.conv2bin(mtx, binp)
    serial = num_check_seq.checksum_of(mtx, 8)
    # definition check against the plain formula
    ref = sum(v * 8 * (r / 1000.0) * (c / 1000.0) for r, c, v in zip(m.rows, m.cols, m.vals))
    assert abs(serial - ref) < 1e-9 * max(1.0, abs(ref))
    out = _torchrun(4, "spcomm3d_b200.cli.num_res_check", "-k", "8", "-c", "2", "--device", "cpu", binp)
    assert out.returncode == 0, out.stderr[-2000:]
    sums = [float(l.rsplit("=", 1)[1]) for l in out.stdout.splitlines() if l.startswith("Global numerical sum") and "sddmm" in l]
    assert len(sums) == 2 and all(abs(s - serial) < 1e-6 * max(1.0, abs(serial)) for s in sums)


def test_single_process_tools(tmp_path):
    from spcomm3d_b200.cli import count_excess, read_distribute, serial_sim
    m = generate.fixed_degree(200, 200, 3, seed=2)
    p = str(tmp_path / "g.bin")
    binfmt.write_bin(p, m)
    serial_sim.main(["-n", "4,16", "-m", p])
    count_excess.main([p, "-n", "16"])
    count_excess.main([p, "--empty"])
    read_distribute.main([p, "-x", "2", "-y", "2", "-o", str(tmp_path / "blk")])
    total = sum(binfmt.read_bin_header(str(tmp_path / f"blk_{x}_{y}.bin"))[2] for x in range(2) for y in range(2))
    assert total == m.nnz


def test_gpu_runtimes_start_a_group_with_a_host_backend(monkeypatch):
    """The collective .bin reader exchanges host arrays; on GPU ranks the group must therefore carry gloo next
    to NCCL.  Checked on the call the runtime makes (no GPU needed)."""
    import argparse
    import torch.distributed as dist
    from spcomm3d_b200.cli import common
    seen = {}
    monkeypatch.setenv("WORLD_SIZE", "2")
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setattr(common.torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(common.torch.cuda, "set_device", lambda d: None)

    def fake_init(backend, **kw):
        seen["backend"], seen["kw"] = backend, kw
        raise RuntimeError("stop here")

    monkeypatch.setattr(dist, "init_process_group", fake_init)
    args = argparse.Namespace(device=None, mesh=None, Z=1, dtype=None)
    with pytest.raises(RuntimeError, match="stop here"):
        common.Runtime(args)
    assert seen["backend"] == "cpu:gloo,cuda:nccl" and "device_id" in seen["kw"]


def test_serial_sim_reference_line_layout(tmp_path, capsys):
    """--ref-format: `name rows cols nnz N XxYxZ f c S|B 4 averages 4 integer maxima` (miniapp/serialSim.cpp:
    227-230, 249-252), X <= Y as its findXY picks them, the dense line counted message by message, and the
    density sweep 1e-7 ... 1e-3 under the name SYNTH (:278-287)."""
    from spcomm3d_b200.cli import serial_sim
    serial_sim.main(["-n", "16,32", "-i", "3000", "--density-sweep", "--ref-format", "-c", "2", "-k", "64"])
    lines = [l.split() for l in capsys.readouterr().out.splitlines() if l and not l.startswith("#")]
    assert len(lines) == 5 * 2 * 2
    nnz_seen = set()
    for t in lines:
        assert len(t) == 17 and t[0] == "SYNTH" and t[1] == t[2] == "3000" and t[8] in ("S", "B")
        N, (X, Y, Z) = int(t[4]), (int(v) for v in t[5].split("x"))
        assert X * Y * Z == N and X <= Y and Z == 2 and t[6] == "64" and t[7] == "2"
        assert all("." in v for v in t[9:13]) and all(v.isdigit() for v in t[13:17])
        nnz_seen.add(int(t[3]))
        if t[8] == "B":   # every rank sends to, and hears from, the X + Y - 2 other ranks of its two lines
            assert float(t[9]) == float(t[11]) == X + Y - 2 and t[13] == t[15] == str(X + Y - 2)
    assert sorted(nnz_seen) == [int(3000 * 3000 * 10.0 ** e) for e in range(-7, -2)]


# ---- failure detection, all on the host -------------------------------------
def _absent_peer(rank, world):
    """Rank 1 never joins the exchange; rank 0's collective must end with an
    error after the group's timeout instead of hanging."""
    import torch.distributed as dist
    from spcomm3d_b200.models.dist_ops import DistSpMM
    from spcomm3d_b200.parallel.mesh import Mesh3D, MeshGroups
    from spcomm3d_b200.parallel.plan import build_my_plan
    mesh = Mesh3D(2, 1, 1)
    groups = MeshGroups.create(mesh)
    m = generate.fixed_degree(100, 100, 3, seed=1)
    _, plan = build_my_plan(m, mesh, rank, seed=1)
    op = DistSpMM(plan, groups, 8, torch.float64, "cpu", "sparseNRB")
    op.run()  # one healthy step
    if rank == 1:
        return  # leaves between steps
    with pytest.raises(Exception):
        op.run()


def _entry_short_timeout(rank, world, port, fn):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    fn(rank, world)


def test_absent_peer_ends_in_an_error_not_a_hang():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    port = free_port()
    procs = [ctx.Process(target=_entry_short_timeout, args=(r, 2, port, _absent_peer)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(not p.is_alive() for p in procs)
    assert procs[0].exitcode == 0, "rank 0 should have caught the timeout error"


def _heartbeat_and_fingerprint(rank, world):
    from spcomm3d_b200.parallel import health
    from spcomm3d_b200.parallel.mesh import Mesh3D, MeshGroups
    from spcomm3d_b200.parallel.plan import build_my_plan
    mesh = Mesh3D(2, 1, 1)
    groups = MeshGroups.create(mesh)
    m = generate.fixed_degree(100, 100, 3, seed=1)
    _, plan = build_my_plan(m, mesh, rank, seed=1)
    health.check_consistent(plan, groups)
    # rank 1 plans a different matrix: everyone must be told
    _, wrong = build_my_plan(generate.fixed_degree(100, 100, 4, seed=1) if rank == 1 else m, mesh, rank, seed=1)
    with pytest.raises(ValueError, match="not consistent"):
        health.check_consistent(wrong, groups)
    hb = health.Heartbeat(rank, world)
    import torch.distributed as dist
    dist.barrier()
    hb.beat(1)
    hb.require_alive(1, wait_s=10)
    if rank == 0:
        hb.beat(2)
        with pytest.raises(health.RankFailure, match=r"\[1\]"):
            hb.require_alive(2, wait_s=0.5)  # rank 1 never reports step 2


def test_plan_fingerprint_and_heartbeat():
    run_ranks(_heartbeat_and_fingerprint, 2)


def test_numa_placement_from_a_fake_sysfs(tmp_path):
    """The rank is restricted to the CPUs of its GPU's NUMA node; unknown node or device: nothing changes."""
    import os
    from spcomm3d_b200.utils import affinity
    assert affinity.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    pci = "0000:1b:00.0"
    (tmp_path / "bus/pci/devices" / pci).mkdir(parents=True)
    (tmp_path / "bus/pci/devices" / pci / "numa_node").write_text("1\n")
    mine = sorted(os.sched_getaffinity(0))
    (tmp_path / "devices/system/node/node1").mkdir(parents=True)
    (tmp_path / "devices/system/node/node1/cpulist").write_text(",".join(str(c) for c in mine) + ",100000\n")
    info = affinity.bind_near(pci, sysfs=str(tmp_path), apply=False)
    assert info == {"node": 1, "cpus": len(mine)}
    if len(mine) >= 2:
        half = affinity.bind_near(pci, sysfs=str(tmp_path), slot=1, nslots=2, apply=False)
        assert half["cpus"] == len(mine) // 2
    assert affinity.bind_near("0000:ff:00.0", sysfs=str(tmp_path), apply=False)["node"] is None
    (tmp_path / "bus/pci/devices" / pci / "numa_node").write_text("-1\n")
    assert affinity.bind_near(pci, sysfs=str(tmp_path), apply=False)["node"] is None
    assert affinity.bind_near(None)["node"] is None


def test_cpu_affinity_from_a_fake_nvml(monkeypatch):
    """Without a NUMA node in sysfs the CPUs close to the GPU come from the driver's affinity mask."""
    import os
    import types
    import torch
    from spcomm3d_b200.utils import affinity

    class FakeNvml:
        def nvmlDeviceGetHandleByUUID(self, uuid):
            assert uuid == "GPU-1234"
            return "h"

        def nvmlDeviceGetCpuAffinity(self, handle, nwords):
            return [0b1010] + [0] * (nwords - 2) + ([1] if nwords > 1 else [])

    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda i: types.SimpleNamespace(uuid="1234"))
    cpus = affinity.nvml_cpu_affinity(0, nvml=FakeNvml())
    nwords = ((os.cpu_count() or 64) + 63) // 64
    assert cpus == ({1, 3} | ({64 * (nwords - 1)} if nwords > 1 else set()))
    mine = sorted(os.sched_getaffinity(0))
    assert affinity.bind_to(set(mine), apply=False) == len(mine)
    assert affinity.bind_to({10 ** 6}, apply=False) == 0 and affinity.bind_to(set()) == 0


def test_ranks_are_spread_over_the_visible_gpus(monkeypatch):
    """Fewer ranks than GPUs: rank r runs on device r * visible / world, so that neighbouring ranks do not
    share a PCIe uplink; SP3_DEVICE_MAP=dense or a count that does not divide keeps rank r on device r."""
    import importlib.util
    import pathlib
    import torch
    spec = importlib.util.spec_from_file_location("sp3_bench", pathlib.Path(__file__).resolve().parent.parent / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 8)
    monkeypatch.delenv("SP3_DEVICE_MAP", raising=False)
    assert [bench.pick_device(r, 4) for r in range(4)] == [0, 2, 4, 6]
    assert [bench.pick_device(r, 2) for r in range(2)] == [0, 4]
    assert [bench.pick_device(r, 8) for r in range(8)] == list(range(8))
    assert [bench.pick_device(r, 3) for r in range(3)] == [0, 1, 2]
    monkeypatch.setenv("SP3_DEVICE_MAP", "dense")
    assert [bench.pick_device(r, 4) for r in range(4)] == [0, 1, 2, 3]
