"""Local sm_100a kernels against plain PyTorch references (fp32 kernels vs an
fp32/fp64 torch restatement of the same op)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _csr(nrows, ncols, degs, seed):
    g = torch.Generator().manual_seed(seed)
    rowptr = torch.zeros(nrows + 1, dtype=torch.int64)
    rowptr[1:] = torch.cumsum(torch.as_tensor(degs, dtype=torch.int64), 0)
    nnz = int(rowptr[-1])
    rowidx = torch.repeat_interleave(torch.arange(nrows), torch.as_tensor(degs)).int()
    colidx = torch.randint(0, ncols, (nnz,), generator=g).int()
    vals = torch.rand(nnz, generator=g, dtype=torch.float64)
    return rowptr, rowidx, colidx, vals


def _degs(nrows, seed, heavy=True):
    rng = np.random.default_rng(seed)
    d = rng.poisson(6, nrows)
    d[rng.integers(0, nrows, nrows // 10)] = 0
    if heavy:
        d[rng.integers(0, nrows, 3)] = [700, 1300, 2049]
    return d


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float64, 1e-12)])
@pytest.mark.parametrize("k", [4, 8, 32, 64, 128, 256, 20, 7, 512])
def test_sddmm(dtype, tol, k):
    from spcomm3d_b200.ops import local
    nrows, ncols = 3000, 2500
    rowptr, rowidx, colidx, vals = _csr(nrows, ncols, _degs(nrows, 1), 2)
    g = torch.Generator().manual_seed(3)
    A = torch.randn(nrows, k, generator=g, dtype=torch.float64)
    B = torch.randn(ncols, k, generator=g, dtype=torch.float64)
    ref = (A[rowidx.long()] * B[colidx.long()]).sum(1) * vals
    out = local.sddmm(rowidx.cuda(), colidx.cuda(), vals.to(dtype).cuda(), A.to(dtype).cuda(), B.to(dtype).cuda())
    scale = ref.abs().max()
    assert (out.cpu().double() - ref).abs().max() <= tol * scale * max(1, k ** 0.5)
    out2 = local.sddmm(rowidx.cuda(), colidx.cuda(), None, A.to(dtype).cuda(), B.to(dtype).cuda())
    ref2 = (A[rowidx.long()] * B[colidx.long()]).sum(1)
    assert (out2.cpu().double() - ref2).abs().max() <= tol * ref2.abs().max() * max(1, k ** 0.5)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float64, 1e-12)])
@pytest.mark.parametrize("k", [4, 32, 64, 128, 256, 20, 7])
@pytest.mark.parametrize("beta", [0.0, 1.0, 0.5])
def test_spmm(dtype, tol, k, beta):
    from spcomm3d_b200.ops import cuda_ops, local
    nrows, ncols = 3000, 2500
    rowptr, rowidx, colidx, vals = _csr(nrows, ncols, _degs(nrows, 4), 5)
    g = torch.Generator().manual_seed(6)
    X = torch.randn(ncols, k, generator=g, dtype=torch.float64)
    Y0 = torch.randn(nrows, k, generator=g, dtype=torch.float64)
    ref = beta * Y0
    ref.index_add_(0, rowidx.long(), X[colidx.long()] * vals[:, None])
    dev = "cuda"
    sched = cuda_ops.SpmmSchedule(rowptr.to(dev))
    assert sched.nlong == 3
    Y = Y0.to(dtype).to(dev)
    local.spmm(rowptr.to(dev), rowidx.to(dev), colidx.to(dev), vals.to(dtype).to(dev), X.to(dtype).to(dev), Y, beta,
               sched)
    scale = ref.abs().max()
    assert (Y.cpu().double() - ref).abs().max() <= tol * scale * 8
    # same inputs, second launch: bitwise identical (no atomics on values)
    Y2 = Y0.to(dtype).to(dev)
    local.spmm(rowptr.to(dev), rowidx.to(dev), colidx.to(dev), vals.to(dtype).to(dev), X.to(dtype).to(dev), Y2, beta,
               sched)
    assert torch.equal(Y, Y2)
    assert int(sched.counters.abs().sum()) == 0


def test_spmm_padded_leading_dimension():
    from spcomm3d_b200.ops import cuda_ops, local
    nrows, ncols, k, ld = 500, 400, 24, 32
    rowptr, rowidx, colidx, vals = _csr(nrows, ncols, _degs(nrows, 7, heavy=False), 8)
    X = torch.randn(ncols, ld, dtype=torch.float32, device="cuda")
    Y = torch.full((nrows, ld), 7.0, dtype=torch.float32, device="cuda")
    local.spmm(rowptr.cuda(), rowidx.cuda(), colidx.cuda(), vals.float().cuda(), X[:, :k], Y[:, :k], 0.0, None)
    ref = torch.zeros(nrows, k, dtype=torch.float64)
    ref.index_add_(0, rowidx.long(), X[:, :k].cpu().double()[colidx.long()] * vals[:, None])
    assert (Y[:, :k].cpu().double() - ref).abs().max() < 1e-4
    assert torch.all(Y[:, k:] == 7.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("k", [64, 20, 3])
def test_rows(dtype, k):
    from spcomm3d_b200.ops import local
    n, m = 1000, 4000
    g = torch.Generator().manual_seed(9)
    idx = torch.randperm(m, generator=g)[:n].cuda()
    src = torch.randn(m, k, generator=g, dtype=dtype).cuda()
    dst = torch.zeros(n, k, dtype=dtype, device="cuda")
    local.gather_rows(idx, src, dst)
    assert torch.equal(dst, src[idx])
    back = torch.zeros(m, k, dtype=dtype, device="cuda")
    local.scatter_rows(idx, dst, back)
    assert torch.equal(back[idx], dst)
    acc = torch.ones(m, k, dtype=dtype, device="cuda")
    local.scatter_add_rows(idx, dst, acc)
    ref = torch.ones(m, k, dtype=dtype, device="cuda")
    ref[idx] += dst
    assert torch.equal(acc, ref)


def test_fill_rows_matches_host():
    from spcomm3d_b200.ops import cuda_ops
    from spcomm3d_b200.utils import generate
    gids = torch.tensor([0, 5, 17, 123456], dtype=torch.int64)
    host = generate.fill_rows(gids.numpy(), 128, 32, 48, seed=3, stream=2, dtype=np.float32)
    out = torch.zeros(4, 48, dtype=torch.float32, device="cuda")
    cuda_ops.fill_rows(gids.cuda(), 128, 32, out, seed=3, stream=2)
    assert np.abs(out.cpu().numpy() - host).max() < 1e-5
    out1 = torch.zeros(4, 48, dtype=torch.float64, device="cuda")
    cuda_ops.fill_rows(gids.cuda(), 128, 32, out1, kind=generate.FILL_GID_OVER_1000)
    assert float(out1[3, 0]) == 123.456


def test_checksum_and_index_kernels():
    from spcomm3d_b200.ops import cuda_ops
    x = torch.randn(1_000_003, dtype=torch.float32, device="cuda")
    s = cuda_ops.checksum(x)
    assert abs(float(s) - float(x.double().sum())) < 1e-6 * x.numel() ** 0.5
    assert torch.equal(s, cuda_ops.checksum(x))
    perm = torch.randperm(1000, device="cuda")
    inv = cuda_ops.invert_perm(perm)
    assert torch.equal(inv[perm], torch.arange(1000, device="cuda"))
    table = torch.arange(100, 200, dtype=torch.int32, device="cuda")
    idx = torch.randint(0, 100, (5000,), dtype=torch.int32, device="cuda")
    assert torch.equal(cuda_ops.remap_indices(idx, table), table[idx.long()])
    st = cuda_ops.new_status("cuda")
    bad = torch.tensor([1, 2, 100], dtype=torch.int32, device="cuda")
    out = cuda_ops.remap_indices(bad, table, st)
    assert st.tolist()[0] == 1 and int(out[2]) == -1  # reported, not faulted


def test_single_gpu_models_match_oracle():
    from spcomm3d_b200.models.dist_ops import DistSDDMM, DistSpMM
    from spcomm3d_b200.ops import oracle
    from spcomm3d_b200.parallel.mesh import Mesh3D
    from spcomm3d_b200.parallel.plan import build_all_plans
    from spcomm3d_b200.utils import generate
    m = generate.zipf_rows(4096, 8192, dmax=1500, seed=1)
    _, plans = build_all_plans(m, Mesh3D(1, 1, 1), seed=2)
    p, k = plans[0], 64
    A = generate.fill_rows(np.arange(m.nrows), k, 0, k, seed=5, stream=1, dtype=np.float64)
    B = generate.fill_rows(np.arange(m.ncols), k, 0, k, seed=5, stream=2, dtype=np.float64)
    op = DistSDDMM(p, None, k, torch.float32, "cuda")
    op.fill_owned(op.A_owned, p.row.owned_gids, seed=5, stream=1)
    op.fill_owned(op.B_owned, p.col.owned_gids, seed=5, stream=2)
    c = op.run()
    ref = oracle.sddmm_ref(m, A, B)
    got = torch.empty(m.nnz, dtype=torch.float64)
    got[torch.from_numpy(p.src_perm)] = c.cpu().double()
    assert (got - ref).abs().max() < 1e-4 * ref.abs().max()
    sp = DistSpMM(p, None, k, torch.float32, "cuda")
    sp.fill_owned(sp.X_owned, p.col.owned_gids, seed=5, stream=2)
    y = sp.run()
    yref = oracle.spmm_ref(m, B)[p.row.owned_gids]
    assert (y.cpu().double() - yref).abs().max() < 1e-4 * yref.abs().max()


@pytest.mark.parametrize("k", [8, 32, 64, 128, 256, 24])
def test_sddmm_tma_gather(k):
    """B rows staged by TMA tile::gather4 copies; same result as the fp64 reference."""
    from spcomm3d_b200.ops import cuda_ops
    nrows, ncols = 3000, 2500
    rowptr, rowidx, colidx, vals = _csr(nrows, ncols, _degs(nrows, 1), 2)
    g = torch.Generator().manual_seed(3)
    A = torch.randn(nrows, k, generator=g, dtype=torch.float64)
    B = torch.randn(ncols, k, generator=g, dtype=torch.float64)
    ref = (A[rowidx.long()] * B[colidx.long()]).sum(1) * vals
    st = cuda_ops.new_status("cuda")
    out = torch.full((rowidx.shape[0],), float("nan"), dtype=torch.float32, device="cuda")
    cuda_ops.sddmm_tma(rowidx.cuda(), colidx.cuda(), vals.float().cuda(), A.float().cuda(), B.float().cuda(), out, st)
    torch.cuda.synchronize()
    assert st.tolist()[0] == 0, st.tolist()
    assert (out.cpu().double() - ref).abs().max() <= 2e-5 * ref.abs().max() * k ** 0.5


@pytest.mark.parametrize("k", [8, 32, 64, 128, 256, 24])
def test_spmm_tma_gather(k):
    """X rows staged by TMA tile::gather4 copies; rows with zero, few and thousands of nonzeros; beta."""
    from spcomm3d_b200.ops import cuda_ops
    nrows, ncols = 3000, 2500
    rowptr, rowidx, colidx, vals = _csr(nrows, ncols, _degs(nrows, 1), 2)
    g = torch.Generator().manual_seed(3)
    X = torch.randn(ncols, k, generator=g, dtype=torch.float64)
    Y0 = torch.randn(nrows, k, generator=g, dtype=torch.float64)
    S = torch.sparse_coo_tensor(torch.stack([rowidx.long(), colidx.long()]), vals, (nrows, ncols)).coalesce()
    prod = torch.sparse.mm(S, X)
    st = cuda_ops.new_status("cuda")
    for beta in (0.0, 0.5):
        Y = Y0.float().cuda() if beta else torch.full((nrows, k), float("nan"), dtype=torch.float32, device="cuda")
        cuda_ops.spmm_tma(rowidx.cuda(), colidx.cuda(), vals.float().cuda(), X.float().cuda(), Y, beta, st)
        torch.cuda.synchronize()
        assert st.tolist()[0] == 0, st.tolist()
        ref = prod + beta * Y0
        assert (Y.cpu().double() - ref).abs().max() <= 2e-5 * ref.abs().max() * 8


@pytest.mark.parametrize("k", [32, 64, 128])
def test_sddmm_dense_panels_on_tensor_cores(k):
    """Hub block x hub columns goes through tcgen05 TF32 tiles, the rest through the gather kernel."""
    from spcomm3d_b200.ops.panel import PanelSDDMM
    rng = np.random.default_rng(5)
    nrows, ncols = 1000, 900
    # a dense corner (rows 0..255 x 100 hub columns, 30 % filled) plus a sparse background
    hub_cols = rng.choice(ncols, 100, replace=False)
    rr, cc = np.nonzero(rng.random((256, 100)) < 0.3)
    rows = np.concatenate([rr, rng.integers(0, nrows, 6000)])
    cols = np.concatenate([hub_cols[cc], rng.integers(0, ncols, 6000)])
    keys = np.unique(rows.astype(np.int64) * ncols + cols)
    rows, cols = (keys // ncols).astype(np.int32), (keys % ncols).astype(np.int32)
    vals = rng.random(keys.size)
    op = PanelSDDMM(rows, cols, vals, nrows, ncols)
    assert op.npanels >= 2 and op.n_panel_nnz > 5000 and op.n_panel_nnz + op.n_rest == keys.size
    A = torch.from_numpy(rng.standard_normal((nrows, k))).float()
    B = torch.from_numpy(rng.standard_normal((ncols, k))).float()
    out = torch.full((keys.size,), float("nan"), dtype=torch.float32, device="cuda")
    op.run(A.cuda(), B.cuda(), out)
    torch.cuda.synchronize()
    assert op.status.tolist()[0] == 0, op.status.tolist()
    ref = (A.double()[rows.astype(np.int64)] * B.double()[cols.astype(np.int64)]).sum(1) * torch.from_numpy(vals)
    err = (out.cpu().double() - ref).abs()
    assert not torch.isnan(out).any()
    # TF32 operands: ~2^-11 relative per product, sqrt(k) growth
    assert err.max() <= 4e-3 * k ** 0.5
    # the remainder went through the fp32 kernel and is tight
    rest = op.r_pos.cpu().long()
    assert err[rest].max() <= 2e-5 * max(1.0, ref.abs().max()) * k ** 0.5


@pytest.mark.parametrize("k", [32, 64, 128, 256])
def test_spmm_dense_panels_on_tensor_cores(k):
    """Panels of a hub block accumulate S_panel @ X in TMEM (tcgen05 TF32); remainder + beta via the gather kernel."""
    from spcomm3d_b200.ops.panel import PanelSpMM
    rng = np.random.default_rng(6)
    nrows, ncols = 1000, 900
    hub_cols = rng.choice(ncols, 150, replace=False)   # three 64-column tiles per block, the last one partial
    rr, cc = np.nonzero(rng.random((300, 150)) < 0.3)  # rows 256..299: a block whose last rows hold no panel nonzeros
    rows = np.concatenate([rr, rng.integers(0, nrows, 6000)])
    cols = np.concatenate([hub_cols[cc], rng.integers(0, ncols, 6000)])
    keys = np.unique(rows.astype(np.int64) * ncols + cols)
    rows, cols = (keys // ncols).astype(np.int32), (keys % ncols).astype(np.int32)
    vals = rng.random(keys.size)
    X = torch.from_numpy(rng.standard_normal((ncols, k))).float()
    Y0 = torch.from_numpy(rng.standard_normal((nrows, k))).float()
    S = torch.sparse_coo_tensor(np.stack([rows, cols]).astype(np.int64), torch.from_numpy(vals), (nrows, ncols))
    # group_panels = 8: one group per row block (plain stores); 2: hub blocks cut into groups (atomic adds)
    for group_panels, beta in ((8, 0.0), (8, 0.5), (2, 0.5)):
        op = PanelSpMM(rows, cols, vals, nrows, ncols, group_panels=group_panels)
        assert op.npanels >= 4 and op.n_panel_nnz > 5000 and op.n_panel_nnz + op.n_rest == keys.size
        assert (op.ngroups > 3 and int(op.grp_shared.sum()) > 0) if group_panels == 2 else int(op.grp_shared.sum()) == 0
        Y = Y0.clone().cuda()
        op.run(X.cuda(), Y, beta)
        torch.cuda.synchronize()
        assert op.status.tolist()[0] == 0, op.status.tolist()
        ref = beta * Y0.double() + torch.sparse.mm(S, X.double())
        err = (Y.cpu().double() - ref).abs()
        assert not torch.isnan(Y).any()
        # TF32 operands: ~2^-11 relative per product; a hub row sums ~45 panel products of size <= 1 * |x|
        assert err.max() <= 2e-2
        # rows without panel nonzeros went through the fp32 kernel only and are tight
        assert err[600:].max() <= 2e-5 * max(1.0, float(ref.abs().max()))

def test_validate_indices_reports_instead_of_faulting():
    from spcomm3d_b200.ops import cuda_ops
    r = torch.tensor([0, 1, 2, 3], dtype=torch.int32, device="cuda")
    c = torch.tensor([0, 5, 9, 2], dtype=torch.int32, device="cuda")
    cuda_ops.validate_indices(r, c, 4, 10)
    with pytest.raises(IndexError, match="column index 9 at nonzero 2"):
        cuda_ops.validate_indices(r, c, 4, 9)
