"""Fused kernels with every rank of a mesh on ONE GPU (LocalFabric): each
rank's heap is a local allocation, peers' pointers are plain device pointers,
and the three kernel phases are launched in lock step so that no launch waits
for a later one.  Checks pointer tables, slice routing, slot routing, the
double-buffered partial buffers (two epochs) and poison-filled staging."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(meshstr, gen, k, seed=3):
    from spcomm3d_b200.parallel.mesh import Mesh3D
    from spcomm3d_b200.parallel.plan import build_all_plans
    from spcomm3d_b200.utils import generate
    mesh = Mesh3D.parse(meshstr)
    m = generate.from_spec(gen, seed=seed)
    _, plans = build_all_plans(m, mesh, seed=seed)
    A = generate.fill_rows(np.arange(m.nrows), k, 0, k, seed=5, stream=1, dtype=np.float64)
    B = generate.fill_rows(np.arange(m.ncols), k, 0, k, seed=5, stream=2, dtype=np.float64)
    return mesh, m, plans, A, B


MESHES = ["2x2x2", "4x2x1", "1x1x8", "2x1x2", "1x2x1", "3x2x1"]


# (pull/compute overlap in waves, push mode of the Z partials: 1 direct, 0 staged + one push at the end, 2 staged +
#  per-ticket, staged A rows, pulls by bulk copies through shared memory instead of vector loads)
@pytest.mark.parametrize("overlap,push,stage_a,bulk", [(True, 1, False, True), (False, 0, True, False),
                                                       (False, 2, False, True), (True, None, False, False),
                                                       (True, 0, True, True), (True, None, None, None)])
@pytest.mark.parametrize("meshstr", MESHES)
@pytest.mark.parametrize("gen,k", [("uniform:600:500:7", 64), ("zipf:700:900:1.6:600", 32)])
def test_fused_sddmm_all_ranks_one_gpu(meshstr, gen, k, overlap, push, stage_a, bulk):
    from spcomm3d_b200.models.dist_ops import DistSDDMM
    from spcomm3d_b200.ops import oracle
    from spcomm3d_b200.ops.fused import FusedSDDMM, run_lockstep
    from spcomm3d_b200.parallel.mesh import split_k
    from spcomm3d_b200.parallel.symm import LocalFabric
    from spcomm3d_b200.utils.sparse import CooMatrix
    mesh, m, plans, A, B = _setup(meshstr, gen, k)
    fabric = LocalFabric(mesh.size)
    kl = [split_k(k, mesh.Z, plans[r].coords[2])[1] for r in range(mesh.size)]
    heaps = fabric.heaps([FusedSDDMM.region_sizes(plans[r], kl[r]) for r in range(mesh.size)])
    ops = [DistSDDMM(plans[r], None, k, torch.float32, "cuda", "fused", heap=heaps[r], timeout_s=2.0,
                     overlap=overlap, direct_push=push, stage_a=stage_a, bulk_pull=bulk)
           for r in range(mesh.size)]
    for epoch in range(2):
        for op in ops:
            p = op.plan
            op.fill_owned(op.A_owned, p.row.owned_gids, seed=5 + epoch, stream=1)
            op.fill_owned(op.B_owned, p.col.owned_gids, seed=5 + epoch, stream=2)
            op.poison_unowned()
        run_lockstep([op._fused for op in ops])
        from spcomm3d_b200.utils import generate
        Ae = generate.fill_rows(np.arange(m.nrows), k, 0, k, seed=5 + epoch, stream=1, dtype=np.float64)
        Be = generate.fill_rows(np.arange(m.ncols), k, 0, k, seed=5 + epoch, stream=2, dtype=np.float64)
        for op in ops:
            op._fused.check()
            p = op.plan
            off, ln = p.owned_nnz_slice()
            pos = op.owned_positions()
            mine = CooMatrix(m.nrows, m.ncols, p.global_rows()[pos], p.global_cols()[pos], p.vals[pos])
            ref = oracle.sddmm_ref(mine, Ae, Be)
            got = op._fused.out[:op._fused.out_len]
            got = got[off:off + ln] if mesh.Z == 1 else got
            assert got.shape[0] == ln
            if ln:
                assert (got.cpu().double() - ref).abs().max() <= 2e-5 * max(1.0, ref.abs().max()) * k ** 0.5


# reduce: "slots" = per-source slots + ordered sum at the owner; "atomic" = adds into the owner's rows (16-byte
# vector atomics, or one 4-byte atomic per value)
@pytest.mark.parametrize("reduce,red_v4,bulk", [("slots", True, True), ("slots", True, False), ("atomic", True, None),
                                                ("atomic", False, False)])
@pytest.mark.parametrize("meshstr", MESHES)
@pytest.mark.parametrize("gen,k", [("uniform:600:500:7", 64), ("zipf:700:900:1.6:600", 32)])
def test_fused_spmm_all_ranks_one_gpu(meshstr, gen, k, reduce, red_v4, bulk):
    from spcomm3d_b200.models.dist_ops import DistSpMM
    from spcomm3d_b200.ops import oracle
    from spcomm3d_b200.ops.fused import FusedSpMM, run_lockstep
    from spcomm3d_b200.parallel.mesh import split_k
    from spcomm3d_b200.parallel.symm import LocalFabric
    from spcomm3d_b200.utils import generate
    mesh, m, plans, A, B = _setup(meshstr, gen, k)
    fabric = LocalFabric(mesh.size)
    kl = [split_k(k, mesh.Z, plans[r].coords[2])[1] for r in range(mesh.size)]
    heaps = fabric.heaps([FusedSpMM.region_sizes(plans[r], kl[r], reduce) for r in range(mesh.size)])
    ops = [DistSpMM(plans[r], None, k, torch.float32, "cuda", "fused", heap=heaps[r], timeout_s=2.0,
                    reduce=reduce, red_v4=red_v4, bulk_pull=bulk)
           for r in range(mesh.size)]
    results = []
    for epoch in range(3):
        beta = 0.0 if epoch < 2 else 0.5
        for op in ops:
            op.fill_owned(op.X_owned, op.plan.col.owned_gids, seed=5 + epoch % 2, stream=2)
            op.poison_unowned()
            if beta == 0.0:
                op.Y_owned.fill_(float("nan"))  # beta = 0 must overwrite, not scale
        prev = [op.Y_owned.clone() for op in ops]
        run_lockstep([op._fused for op in ops], [(op.Y_owned, beta) for op in ops])
        Be = generate.fill_rows(np.arange(m.ncols), k, 0, k, seed=5 + epoch % 2, stream=2, dtype=np.float64)
        full = oracle.spmm_ref(m, Be)
        for op, pv in zip(ops, prev):
            op._fused.check()
            p = op.plan
            ko, kw = split_k(k, mesh.Z, p.coords[2])
            ref = full[p.row.owned_gids][:, ko:ko + kw]
            if beta:
                ref = ref + beta * pv.cpu().double()
            if ref.numel():
                assert (op.Y_owned.cpu().double() - ref).abs().max() <= 2e-5 * max(1.0, ref.abs().max()) * 8
        results.append([op.Y_owned.clone() for op in ops])
    # epochs 0 and 2 use different data; rerun of the same data must be bitwise identical
    for op in ops:
        op.fill_owned(op.X_owned, op.plan.col.owned_gids, seed=5, stream=2)
    run_lockstep([op._fused for op in ops], [(op.Y_owned, 0.0) for op in ops])
    for op, y0 in zip(ops, results[0]):
        if reduce == "slots":
            assert torch.equal(op.Y_owned, y0)
        elif y0.numel():  # atomic adds: the order of the additions may differ between runs
            assert (op.Y_owned - y0).abs().max() <= 1e-5 * max(1.0, float(y0.abs().max()))


@pytest.mark.parametrize("meshstr,k", [("2x2x2", 30), ("1x1x8", 30), ("2x1x2", 7), ("3x2x1", 50)])
def test_fused_kernels_any_inner_dimension(meshstr, k):
    """k / Z that is not a multiple of 4, and k that Z does not divide (fiber ranks then hold slices of
    different widths, as the reference allows: floc = k / Z (+1), miniapp/bench_spmm.cpp:167-172): the dense
    blocks get a leading dimension rounded up to 4 with zero padding."""
    from spcomm3d_b200.models.dist_ops import DistSDDMM, DistSpMM
    from spcomm3d_b200.ops import oracle
    from spcomm3d_b200.ops.fused import FusedSDDMM, FusedSpMM, run_lockstep
    from spcomm3d_b200.parallel.mesh import split_k
    from spcomm3d_b200.parallel.symm import LocalFabric
    from spcomm3d_b200.utils.sparse import CooMatrix
    mesh, m, plans, A, B = _setup(meshstr, "zipf:700:900:1.6:600", k)
    kl = [split_k(k, mesh.Z, plans[r].coords[2])[1] for r in range(mesh.size)]
    assert any(x % 4 for x in kl)
    for cls, F in ((DistSDDMM, FusedSDDMM), (DistSpMM, FusedSpMM)):
        fabric = LocalFabric(mesh.size)
        heaps = fabric.heaps([F.region_sizes(plans[r], kl[r]) for r in range(mesh.size)])
        ops = [cls(plans[r], None, k, torch.float32, "cuda", "fused", heap=heaps[r], timeout_s=2.0)
               for r in range(mesh.size)]
        for op in ops:
            p = op.plan
            if cls is DistSDDMM:
                op.fill_owned(op.A_owned, p.row.owned_gids, seed=5, stream=1)
                op.fill_owned(op.B_owned, p.col.owned_gids, seed=5, stream=2)
            else:
                op.fill_owned(op.X_owned, p.col.owned_gids, seed=5, stream=2)
                op.Y_owned.fill_(float("nan"))
            op.poison_unowned()
        run_lockstep([op._fused for op in ops], [(op.Y_owned, 0.0) for op in ops] if cls is DistSpMM else None)
        full = oracle.spmm_ref(m, B) if cls is DistSpMM else None
        for op in ops:
            op._fused.check()
            p = op.plan
            if cls is DistSDDMM:
                pos = op.owned_positions()
                mine = CooMatrix(m.nrows, m.ncols, p.global_rows()[pos], p.global_cols()[pos], p.vals[pos])
                ref = oracle.sddmm_ref(mine, A, B)
                got = op._fused.out[:op._fused.out_len].cpu().double()
                tol = 2e-5 * max(1.0, float(ref.abs().max()) if ref.numel() else 1.0) * k ** 0.5
            else:
                ko, kw = split_k(k, mesh.Z, p.coords[2])
                ref = full[p.row.owned_gids][:, ko:ko + kw]
                got = op.Y_owned.cpu().double()
                tol = 2e-5 * max(1.0, float(ref.abs().max()) if ref.numel() else 1.0) * 8
            assert got.shape == ref.shape
            if ref.numel():
                assert (got - ref).abs().max() <= tol
        del ops, heaps, fabric


@pytest.mark.parametrize("meshstr,k,reduce", [("2x2x2", 32, "slots"), ("1x1x8", 20, "slots"), ("3x2x1", 33, "atomic"),
                                              ("2x1x2", 64, "slots")])
def test_fused_kernels_fp64(meshstr, k, reduce):
    """The fused kernels in the reference's value type (real_t = double, src/basic.hpp:17), against the fp64
    oracle to fp64 accuracy; run twice, the slot reduction must repeat bit for bit."""
    from spcomm3d_b200.models.dist_ops import DistSDDMM, DistSpMM
    from spcomm3d_b200.ops import oracle
    from spcomm3d_b200.ops.fused import FusedSDDMM, FusedSpMM, run_lockstep
    from spcomm3d_b200.parallel.mesh import split_k
    from spcomm3d_b200.parallel.symm import LocalFabric
    from spcomm3d_b200.utils.sparse import CooMatrix
    mesh, m, plans, A, B = _setup(meshstr, "zipf:700:900:1.6:600", k)
    kl = [split_k(k, mesh.Z, plans[r].coords[2])[1] for r in range(mesh.size)]
    dt = torch.float64
    for cls, F in ((DistSDDMM, FusedSDDMM), (DistSpMM, FusedSpMM)):
        fabric = LocalFabric(mesh.size)
        if cls is DistSpMM:
            heaps = fabric.heaps([F.region_sizes(plans[r], kl[r], reduce, dtype=dt) for r in range(mesh.size)])
            kw = {"reduce": reduce}
        else:
            heaps = fabric.heaps([F.region_sizes(plans[r], kl[r], dtype=dt) for r in range(mesh.size)])
            kw = {}
        ops = [cls(plans[r], None, k, dt, "cuda", "fused", heap=heaps[r], timeout_s=2.0, **kw)
               for r in range(mesh.size)]
        previous = None
        for rep in range(2):
            for op in ops:
                p = op.plan
                if cls is DistSDDMM:
                    op.fill_owned(op.A_owned, p.row.owned_gids, seed=5, stream=1)
                    op.fill_owned(op.B_owned, p.col.owned_gids, seed=5, stream=2)
                else:
                    op.fill_owned(op.X_owned, p.col.owned_gids, seed=5, stream=2)
                    op.Y_owned.fill_(float("nan"))
                op.poison_unowned()
            run_lockstep([op._fused for op in ops], [(op.Y_owned, 0.0) for op in ops] if cls is DistSpMM else None)
            full = oracle.spmm_ref(m, B) if cls is DistSpMM else None
            results = []
            for op in ops:
                op._fused.check()
                p = op.plan
                if cls is DistSDDMM:
                    pos = op.owned_positions()
                    mine = CooMatrix(m.nrows, m.ncols, p.global_rows()[pos], p.global_cols()[pos], p.vals[pos])
                    ref = oracle.sddmm_ref(mine, A, B)
                    got = op._fused.out[:op._fused.out_len].cpu()
                else:
                    ko, kw_ = split_k(k, mesh.Z, p.coords[2])
                    ref = full[p.row.owned_gids][:, ko:ko + kw_]
                    got = op.Y_owned.cpu()
                assert got.dtype == torch.float64 and got.shape == ref.shape
                if ref.numel():
                    assert (got - ref).abs().max() <= 1e-12 * max(1.0, float(ref.abs().max())) * k
                results.append(got.clone())
            if previous is not None and not (cls is DistSpMM and reduce == "atomic"):
                assert all(torch.equal(x, y) for x, y in zip(results, previous))
            previous = results
        del ops, heaps, fabric


def test_atomic_spmm_start_and_main_in_one_launch():
    """Atomic mode with START and MAIN in the same launch (what real ranks run): the rows that receive
    contributions are cleared by START warps with plain stores, and no warp -- of this rank either -- may add
    into them before all START warps are done.  Rank 1's START runs first, alone, so that rank 0 can run START
    and MAIN in one launch without waiting for a later launch; no dense row is pulled on a 1x2x1 mesh, so
    nothing else delays rank 0's MAIN warps."""
    from spcomm3d_b200.models.dist_ops import DistSpMM
    from spcomm3d_b200.ops import oracle
    from spcomm3d_b200.ops.fused import FusedSpMM, PH_FINISH, PH_MAIN, PH_START
    from spcomm3d_b200.parallel.symm import LocalFabric
    from spcomm3d_b200.utils import generate
    k = 64
    mesh, m, plans, A, B = _setup("1x2x1", "zipf:4000:3000:1.5:900", k)
    fabric = LocalFabric(mesh.size)
    heaps = fabric.heaps([FusedSpMM.region_sizes(plans[r], k, "atomic") for r in range(mesh.size)])
    ops = [DistSpMM(plans[r], None, k, torch.float32, "cuda", "fused", heap=heaps[r], timeout_s=2.0,
                    reduce="atomic") for r in range(mesh.size)]
    assert all(op._fused.args.n_recv_x == 0 and op._fused.args.n_crows > 0 for op in ops)
    full = oracle.spmm_ref(m, B)
    for op in ops:
        op.fill_owned(op.X_owned, op.plan.col.owned_gids, seed=5, stream=2)
    for epoch in range(25):
        for op in ops:
            op.Y_owned.fill_(float("nan"))
        f0, f1 = ops[0]._fused, ops[1]._fused
        f1.launch(ops[1].Y_owned, 0.0, phases=PH_START, new_epoch=True)
        f0.launch(ops[0].Y_owned, 0.0, phases=PH_START | PH_MAIN, new_epoch=True)
        f1.launch(ops[1].Y_owned, 0.0, phases=PH_MAIN, new_epoch=False)
        f0.launch(ops[0].Y_owned, 0.0, phases=PH_FINISH, new_epoch=False)
        f1.launch(ops[1].Y_owned, 0.0, phases=PH_FINISH, new_epoch=False)
        for op in ops:
            op._fused.check()
            ref = full[op.plan.row.owned_gids]
            err = (op.Y_owned.cpu().double() - ref).abs().max()
            assert err <= 2e-5 * max(1.0, ref.abs().max()) * 8, (epoch, op.plan.rank, float(err))


def test_wait_runs_out_without_hanging():
    """A flag that nobody sets: the kernel gives up after its limit, records
    where, and the context stays usable."""
    from spcomm3d_b200.models.dist_ops import DistSDDMM
    from spcomm3d_b200.ops.fused import FusedSDDMM, FusedStatusError, PH_MAIN
    from spcomm3d_b200.parallel.mesh import split_k
    from spcomm3d_b200.parallel.symm import LocalFabric
    mesh, m, plans, A, B = _setup("2x1x1", "uniform:300:300:5", 32)
    fabric = LocalFabric(mesh.size)
    heaps = fabric.heaps([FusedSDDMM.region_sizes(plans[r], 32) for r in range(mesh.size)])
    op = DistSDDMM(plans[0], None, 32, torch.float32, "cuda", "fused", heap=heaps[0], timeout_s=0.2)
    # rank 1 never runs its START phase, so rank 0's MAIN phase cannot see READY
    op._fused.launch(phases=PH_MAIN)
    with pytest.raises(FusedStatusError, match="READY"):
        op._fused.check()
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0  # context still healthy
