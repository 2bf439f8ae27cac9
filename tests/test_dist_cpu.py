"""Distributed CPU plumbing: gloo ranks, fp64, every variant against the
single-process oracle, with non-owned rows poisoned before each run."""
import os

import numpy as np
import pytest
import torch

from dist_utils import run_ranks

K = 32


def _check_rank(rank, world, meshstr, kernel, variant, k, from_file):
    from spcomm3d_b200.models.dist_ops import DistSDDMM, DistSpMM
    from spcomm3d_b200.ops import oracle
    from spcomm3d_b200.parallel.mesh import Mesh3D, MeshGroups, split_k
    from spcomm3d_b200.parallel.partition import distribute_from_file
    from spcomm3d_b200.parallel.plan import build_my_plan, build_rank_plan
    from spcomm3d_b200.utils import generate
    from spcomm3d_b200.utils.sparse import CooMatrix

    mesh = Mesh3D.parse(meshstr)
    groups = MeshGroups.create(mesh)
    M, N = 384, 320
    m = generate.fixed_degree(M, N, 6, seed=11)
    if from_file:
        block, directory = distribute_from_file(from_file, mesh, groups, seed=7)
        plan = build_rank_plan(block, directory, groups.coords, gnnz=m.nnz)
    else:
        directory, plan = build_my_plan(m, mesh, rank, seed=7)
    plan.validate()
    directory.check()
    A = generate.fill_rows(np.arange(M), k, 0, k, seed=5, stream=1, dtype=np.float64)
    B = generate.fill_rows(np.arange(N), k, 0, k, seed=5, stream=2, dtype=np.float64)
    z = groups.coords[2]
    if kernel == "sddmm":
        op = DistSDDMM(plan, groups, k, torch.float64, "cpu", variant)
        # "sparse" on a mesh with a plane moves A and B rows in one exchange (not with the p2p transport)
        combined = variant == "sparse" and mesh.xy_size > 1 and os.environ.get("SP3_TRANSPORT", "alltoall") == "alltoall"
        assert (op.exAB is not None) == combined
        op.fill_owned(op.A_owned, plan.row.owned_gids, seed=5, stream=1)
        op.fill_owned(op.B_owned, plan.col.owned_gids, seed=5, stream=2)
        for _ in range(2):
            op.poison_unowned()
            c = op.run()
        off, ln = plan.owned_nnz_slice()
        mine = CooMatrix(M, N, plan.global_rows()[off:off + ln], plan.global_cols()[off:off + ln],
                         plan.vals[off:off + ln])
        ref = oracle.sddmm_ref(mine, A, B)
        assert c.shape[0] == ln
        torch.testing.assert_close(c, ref, rtol=1e-12, atol=1e-12)
    else:
        op = DistSpMM(plan, groups, k, torch.float64, "cpu", variant)
        op.fill_owned(op.X_owned, plan.col.owned_gids, seed=5, stream=2)
        for _ in range(2):
            op.poison_unowned()
            y = op.run()
        ko, kl = split_k(k, mesh.Z, z)
        ref = oracle.spmm_ref(m, B)[plan.row.owned_gids][:, ko:ko + kl]
        torch.testing.assert_close(y, ref, rtol=1e-12, atol=1e-12)


def _check_many(rank, world, meshstr, cases, k, from_file):
    for kernel, variant in cases:
        _check_rank(rank, world, meshstr, kernel, variant, k, from_file)


def test_2x2x2_all_variants():
    cases = [(kern, var) for kern in ("sddmm", "spmm") for var in ("sparse", "sparseNRB", "dense")]
    run_ranks(_check_many, 8, "2x2x2", cases, K, None)


def test_p2p_transport(monkeypatch):
    """One receive and one send per actual neighbour instead of the all-to-all with split sizes."""
    monkeypatch.setenv("SP3_TRANSPORT", "p2p")   # inherited by the spawned ranks
    cases = [(kern, var) for kern in ("sddmm", "spmm") for var in ("sparse", "sparseNRB")]
    run_ranks(_check_many, 6, "3x2x1", cases, 12, None)


@pytest.mark.parametrize("meshstr,k", [("4x2x1", 32), ("1x1x8", 20), ("2x1x2", 7), ("1x3x1", 16), ("3x1x1", 16)])
def test_other_meshes(meshstr, k):
    from spcomm3d_b200.parallel.mesh import Mesh3D
    n = Mesh3D.parse(meshstr).size
    run_ranks(_check_many, n, meshstr, [("sddmm", "sparseNRB"), ("spmm", "sparseNRB"), ("sddmm", "dense"),
                                        ("spmm", "dense")], k, None)


def test_distributed_reader(tmp_path):
    from spcomm3d_b200.utils import binfmt, generate
    m = generate.fixed_degree(384, 320, 6, seed=11)
    path = str(tmp_path / "m.bin")
    binfmt.write_bin(path, m)
    run_ranks(_check_many, 8, "2x2x2", [("sddmm", "sparseNRB"), ("spmm", "sparse")], K, path)


def _config1_rank(rank, world):
    """BASELINE config 1: 4096 x 4096, 16 nonzeros per row, A and B 4096 x 32 fp64 N(0,1), 2x2x2, checked
    element-wise against the serial result; then the attention-style chain on the same mesh."""
    from spcomm3d_b200.models.dist_ops import DistSDDMM
    from spcomm3d_b200.models.layer import GatLayer
    from spcomm3d_b200.ops import oracle
    from spcomm3d_b200.parallel.mesh import Mesh3D, MeshGroups, split_k
    from spcomm3d_b200.parallel.plan import build_my_plan
    from spcomm3d_b200.utils import generate
    from spcomm3d_b200.utils.sparse import CooMatrix
    mesh = Mesh3D(2, 2, 2)
    groups = MeshGroups.create(mesh)
    M = N = 4096
    k = 32
    m = generate.fixed_degree(M, N, 16, seed=1)
    _, plan = build_my_plan(m, mesh, rank, seed=1)
    A = generate.fill_rows(np.arange(M), k, 0, k, seed=2, stream=1, dtype=np.float64)
    B = generate.fill_rows(np.arange(N), k, 0, k, seed=2, stream=2, dtype=np.float64)
    op = DistSDDMM(plan, groups, k, torch.float64, "cpu", "sparseNRB")
    op.fill_owned(op.A_owned, plan.row.owned_gids, seed=2, stream=1)
    op.fill_owned(op.B_owned, plan.col.owned_gids, seed=2, stream=2)
    op.poison_unowned()
    c = op.run()
    off, ln = plan.owned_nnz_slice()
    mine = CooMatrix(M, N, plan.global_rows()[off:off + ln], plan.global_cols()[off:off + ln], plan.vals[off:off + ln])
    torch.testing.assert_close(c, oracle.sddmm_ref(mine, A, B), rtol=1e-12, atol=1e-12)
    # chain: Y = (S o (A B^T)) X with X = B
    layer = GatLayer(plan, groups, k, torch.float64, "cpu", "sparseNRB")
    for o_ in (layer.sddmm,):
        o_.fill_owned(o_.A_owned, plan.row.owned_gids, seed=2, stream=1)
        o_.fill_owned(o_.B_owned, plan.col.owned_gids, seed=2, stream=2)
    layer.spmm.fill_owned(layer.spmm.X_owned, plan.col.owned_gids, seed=2, stream=2)
    y = layer.run()
    scores = oracle.sddmm_ref(m, A, B)
    cm = CooMatrix(M, N, m.rows, m.cols, scores.numpy())
    ko, kw = split_k(k, mesh.Z, groups.coords[2])
    ref = oracle.spmm_ref(cm, B)[plan.row.owned_gids][:, ko:ko + kw]
    torch.testing.assert_close(y, ref, rtol=1e-10, atol=1e-10)


def test_baseline_config1_and_chain():
    run_ranks(_config1_rank, 8)


def _degenerate_rank(rank, world, which):
    import torch.distributed as dist
    from spcomm3d_b200.models.dist_ops import DistSDDMM, DistSpMM
    from spcomm3d_b200.parallel.mesh import Mesh3D, MeshGroups
    from spcomm3d_b200.parallel.plan import build_my_plan
    from spcomm3d_b200.utils.sparse import CooMatrix
    m = [CooMatrix(10, 12, np.zeros(0), np.zeros(0), np.zeros(0), name="empty"),
         CooMatrix(1, 1, [0], [0], [2.0], name="one"),
         CooMatrix(3, 50, [0, 1, 2, 2], [4, 7, 9, 49], [1.0, 2.0, 3.0, 4.0], name="thin")][which]
    mesh = Mesh3D(2, 1, 2)
    groups = MeshGroups.create(mesh)
    _, plan = build_my_plan(m, mesh, rank, seed=1)
    k = 6
    for variant in ("sparse", "sparseNRB", "dense"):
        sd = DistSDDMM(plan, groups, k, torch.float64, "cpu", variant)
        sd.A_owned.fill_(1.0)
        sd.B_owned.fill_(1.0)
        sp = DistSpMM(plan, groups, k, torch.float64, "cpu", variant)
        sp.X_owned.fill_(1.0)
        tot = torch.tensor([float(sd.run().sum()), float(sp.run().sum())], dtype=torch.float64)
        dist.all_reduce(tot)
        # all-ones operands: every nonzero contributes k * value, once over the whole mesh
        assert tot.tolist() == pytest.approx([k * float(m.vals.sum())] * 2), (variant, tot.tolist())


@pytest.mark.parametrize("which", [0, 1, 2])
def test_degenerate_matrices_distributed(which):
    """No nonzeros, a 1 x 1 matrix, fewer rows than ranks: most blocks and exchanges are empty."""
    run_ranks(_degenerate_rank, 4, which)


def _plan_from_own_block(rank, world, meshstr, spec):
    """Every rank generates only its own block of a synthetic matrix; the plan must equal the one built from
    the whole matrix, array for array."""
    from spcomm3d_b200.parallel.mesh import Mesh3D, MeshGroups
    from spcomm3d_b200.parallel.plan import build_my_plan, build_my_plan_from_spec
    from spcomm3d_b200.utils import generate
    mesh = Mesh3D.parse(meshstr)
    groups = MeshGroups.create(mesh)
    _, plan, whole = build_my_plan_from_spec(spec, mesh, groups, seed=7)
    assert whole is None   # the whole matrix was never built
    m = generate.from_spec(spec, seed=7)
    _, ref = build_my_plan(m, mesh, rank, seed=7)
    assert plan.gnnz == ref.gnnz == m.nnz and plan.coords == ref.coords
    for name in ("rowptr", "rowidx", "colidx", "vals"):
        assert np.array_equal(getattr(plan, name), getattr(ref, name)), name
    for side in ("row", "col"):
        for f in ("owned_gids", "local_gids", "recv_counts", "recv_src_idx", "recv_peer", "send_counts", "send_idx",
                  "peer_owned", "push_offset"):
            assert np.array_equal(getattr(getattr(plan, side), f), getattr(getattr(ref, side), f)), (side, f)


@pytest.mark.parametrize("meshstr,spec", [("2x2x1", "er:500:400:5"), ("2x1x2", "zipf:600:800:1.6:200"),
                                          ("1x2x2", "uniform:300:300:4")])
def test_plan_from_own_block_equals_plan_from_whole_matrix(meshstr, spec):
    run_ranks(_plan_from_own_block, 4, meshstr, spec)
