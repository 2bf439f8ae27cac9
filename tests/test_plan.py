"""Plan properties on virtual meshes: ownership, exactness of the need lists
(volume == brute-force need-set count), layouts, persistence."""
import itertools

import numpy as np
import pytest

from spcomm3d_b200.parallel.mesh import Mesh3D
from spcomm3d_b200.parallel.partition import Directory
from spcomm3d_b200.parallel.plan import RankPlan, build_all_plans
from spcomm3d_b200.parallel import virtual
from spcomm3d_b200.utils import generate
from spcomm3d_b200.utils.sparse import CooMatrix


def _factorizations(n):
    return [(x, y, z) for x, y, z in itertools.product(range(1, n + 1), repeat=3) if x * y * z == n]


def _matrices():
    yield generate.fixed_degree(120, 90, 4, seed=1)
    yield generate.zipf_rows(150, 400, alpha=1.5, dmax=200, seed=2)
    # empty rows, empty columns, an empty block region
    yield CooMatrix(40, 50, [0, 0, 3, 39, 17], [1, 49, 1, 0, 20], np.ones(5), name="tiny")
    yield CooMatrix(30, 30, [], [], [], name="empty")


@pytest.mark.parametrize("n", [1, 2, 4, 8])
def test_plans_for_every_mesh_shape(n):
    for m in _matrices():
        for (X, Y, Z) in _factorizations(n):
            mesh = Mesh3D(X, Y, Z)
            d, plans = build_all_plans(m, mesh, seed=5)
            d.check()
            assert len(plans) == n
            # every id has exactly one owner, inside its mesh line
            assert int(d.row_counts.sum()) == m.nrows and int(d.col_counts.sum()) == m.ncols
            total_nnz = 0
            for r, p in plans.items():
                p.validate()
                x, y, z = p.coords
                if z == 0:
                    total_nnz += p.nnz
                # brute force need sets from the block's own nonzeros
                rows, cols = p.global_rows(), p.global_cols()
                assert (d.rowmap[rows] == x).all() and (d.colmap[cols] == y).all()
                for side, ids, owner in ((p.row, rows, d.row_owner), (p.col, cols, d.col_owner)):
                    need = np.unique(ids)
                    mine = need[owner[need] == side.me]
                    other = need[owner[need] != side.me]
                    assert set(mine) <= set(side.owned_gids)
                    assert sorted(other) == sorted(side.local_gids[side.n_owned:])  # exactly the needed rows
                    assert (np.diff(side.owned_gids) > 0).all()
                    # needed rows grouped by ascending owner, ascending id inside a group
                    off = side.recv_offsets()
                    for q in range(side.npeers):
                        seg = side.local_gids[side.n_owned + off[q]: side.n_owned + off[q + 1]]
                        assert (owner[seg] == q).all() and (np.diff(seg) > 0).all()
            assert total_nnz == m.nnz
            # send lists mirror receive lists
            for r, p in plans.items():
                x, y, z = p.coords
                for q in range(mesh.Y):
                    if q != y:
                        other = plans[mesh.rank_of(x, q, z)]
                        assert other.row.send_counts[y] == p.row.recv_counts[q]
                for q in range(mesh.X):
                    if q != x:
                        other = plans[mesh.rank_of(q, y, z)]
                        assert other.col.send_counts[x] == p.col.recv_counts[q]


def test_respect_comm_never_moves_more_than_random_ownership():
    m = generate.fixed_degree(2000, 2000, 5, seed=3)
    mesh = Mesh3D(4, 4, 1)
    _, a = build_all_plans(m, mesh, seed=1, policy="respect_comm")
    _, b = build_all_plans(m, mesh, seed=1, policy="random")
    va = sum(p.expand_rows()[1] for p in a.values())
    vb = sum(p.expand_rows()[1] for p in b.values())
    assert va < vb


def test_sparse_volume_not_above_dense_volume_and_sim_agrees():
    m = generate.fixed_degree(3000, 2500, 6, seed=4)
    mesh = Mesh3D(4, 2, 1)
    _, plans = build_all_plans(m, mesh, seed=9)
    sim = virtual.serial_sim(m, 4, 2, seed=9)
    recv = [p.expand_rows()[1] for p in plans.values()]
    send = [p.expand_rows()[0] for p in plans.values()]
    assert np.isclose(sim["sparse"]["avgRecvVol"], np.mean(recv)) and sim["sparse"]["maxRecvVol"] == max(recv)
    assert np.isclose(sim["sparse"]["avgSendVol"], np.mean(send)) and sim["sparse"]["maxSendVol"] == max(send)
    assert sim["sparse"]["avgRecvVol"] <= sim["dense"]["avgRecvVol"]
    ex = virtual.count_excess(m, 4, 2, seed=9)
    assert ex["excess_rows"] >= 0 and ex["stored_rows"] == 2 * (m.nrows * 2 + m.ncols * 4) / 2


def test_large_virtual_mesh_simulation():
    m = CooMatrix.random_unique(5000, 5000, 25000, seed=1)
    X, Y = virtual.find_xy(1024)
    assert (X, Y) == (32, 32)
    s = virtual.serial_sim(m, 181, 181, seed=2, policy="random", mode="spmm_pre")
    assert s["sparse"]["avgRecvVol"] <= s["dense"]["avgRecvVol"]
    assert virtual.count_empty(m)[0] > 0


def test_plan_save_load(tmp_path):
    m = generate.fixed_degree(200, 150, 5, seed=1)
    _, plans = build_all_plans(m, Mesh3D(2, 2, 2), seed=2)
    p = plans[5]
    path = str(tmp_path / "plan5")
    p.save(path)
    q = RankPlan.load(path)
    assert q.coords == p.coords and str(q.mesh) == "2x2x2" and q.gnnz == p.gnnz and q.name == p.name
    for f in ("rowptr", "rowidx", "colidx", "vals", "src_perm"):
        assert np.array_equal(getattr(p, f), getattr(q, f))
    for side in ("row", "col"):
        for f in ("owned_gids", "local_gids", "recv_counts", "recv_src_idx", "send_idx", "push_offset"):
            assert np.array_equal(getattr(getattr(p, side), f), getattr(getattr(q, side), f))


def test_directory_is_deterministic_and_seeded():
    m = generate.fixed_degree(300, 300, 4, seed=1)
    a = Directory.from_global(m, Mesh3D(2, 2, 1), seed=3)
    b = Directory.from_global(m, Mesh3D(2, 2, 1), seed=3)
    c = Directory.from_global(m, Mesh3D(2, 2, 1), seed=4)
    assert np.array_equal(a.rowmap, b.rowmap) and np.array_equal(a.row_owner, b.row_owner)
    assert not np.array_equal(a.rowmap, c.rowmap)
    assert np.array_equal(a.rpvec() // 2, a.rowmap)  # owner's mesh row is the row's mesh row


@pytest.mark.parametrize("meshstr", ["1x1x1", "2x2x2", "4x2x1", "1x1x8", "3x1x2"])
def test_degenerate_matrices(meshstr):
    """No nonzeros at all, a 1 x 1 matrix, fewer rows than mesh rows: plans build, blocks may be empty, and the
    CPU kernels accept them."""
    import torch
    from spcomm3d_b200.ops import local
    cases = [CooMatrix(10, 12, np.zeros(0), np.zeros(0), np.zeros(0)),
             CooMatrix(1, 1, [0], [0], [2.0]),
             CooMatrix(3, 50, [0, 1, 2, 2], [4, 7, 9, 49], [1.0, 2.0, 3.0, 4.0])]
    mesh = Mesh3D.parse(meshstr)
    for m in cases:
        _, plans = build_all_plans(m, mesh, seed=1)
        assert sum(p.nnz for p in plans.values()) == m.nnz * mesh.Z
        total = 0.0
        for p in plans.values():
            k = 8
            A = torch.ones(p.row.n_local, k, dtype=torch.float64)
            B = torch.ones(p.col.n_local, k, dtype=torch.float64)
            c = local.sddmm(torch.from_numpy(p.rowidx), torch.from_numpy(p.colidx), torch.from_numpy(p.vals), A, B)
            y = torch.zeros(p.row.n_local, k, dtype=torch.float64)
            local.spmm(torch.from_numpy(p.rowptr), torch.from_numpy(p.rowidx), torch.from_numpy(p.colidx),
                       torch.from_numpy(p.vals), B, y, 0.0)
            if p.coords[2] == 0:
                total += float(c.sum())
        assert total == pytest.approx(8 * float(m.vals.sum()))


def test_spmm_wave_items_cover_every_nonzero_once_in_class_order():
    """Work items of the wave-gated SpMM: the re-ordering stays inside rows, long rows are cut into pieces of
    one class each, every nonzero belongs to exactly one item, items come in non-decreasing class order and the
    per-class counts are their prefix sums."""
    from spcomm3d_b200.ops.cuda_ops import PIECE_SHIFT, build_spmm_items, build_spmm_wave_items
    rng = np.random.default_rng(0)
    nrows = 3000
    deg = rng.poisson(4, nrows)
    deg[rng.choice(nrows, 6, replace=False)] = [700, 1300, 513, 2500, 600, 900]
    rowptr = np.zeros(nrows + 1, np.int64)
    rowptr[1:] = np.cumsum(deg)
    nnz = int(rowptr[-1])
    cls = rng.integers(0, 4, nnz).astype(np.int8)
    perm, items, first, npieces, class_items = build_spmm_wave_items(rowptr, cls, 4, long_row=512)
    assert sorted(perm.tolist()) == list(range(nnz))
    rows_of = np.repeat(np.arange(nrows), deg)
    assert np.array_equal(rows_of[perm], rows_of)           # nonzeros stay in their rows
    cp = cls[perm]
    cover = np.zeros(nnz, np.int64)
    last, seen_pieces, per_class = -1, set(), np.zeros(4, np.int64)
    for it in items:
        if it[3] < 0:
            b, e = rowptr[it[0]], rowptr[it[1]]
            c = int(cp[b:e].max()) if e > b else 0
        else:
            b, e = int(it[1]), int(it[2])
            c = int(cp[b:e].max())
            assert cp[b:e].min() == c and 0 < e - b <= 512 and rowptr[it[0]] <= b < e <= rowptr[it[0] + 1]
            lr, pn = it[3] & ((1 << PIECE_SHIFT) - 1), it[3] >> PIECE_SHIFT
            assert pn < npieces[lr] and (lr, pn) not in seen_pieces
            seen_pieces.add((lr, pn))
        cover[b:e] += 1
        assert c >= last
        last = c
        per_class[c] += 1
    assert (cover == 1).all()
    assert np.array_equal(np.cumsum(per_class), class_items)
    assert len(seen_pieces) == int(npieces.sum()) and np.array_equal(first, np.cumsum(npieces) - npieces)
    # the plain schedule numbers its pieces the same way
    it2, f2, n2 = build_spmm_items(rowptr, long_row=512)
    pieces = it2[it2[:, 3] >= 0]
    got = sorted((int(w) & ((1 << PIECE_SHIFT) - 1), int(w) >> PIECE_SHIFT) for w in pieces[:, 3])
    assert got == sorted((lr, j) for lr in range(len(n2)) for j in range(int(n2[lr])))


def test_pull_order_starts_at_the_next_peer_of_the_line(monkeypatch):
    """Ranks of a mesh line pull from different owners at any one time: rank m starts with peer m + 1."""
    import types
    from spcomm3d_b200.ops.fused import _tiles_by_peer_distance
    npeers, tile_rows = 4, 8
    counts = {0: 40, 1: 24, 3: 16}                       # rows needed from each peer by rank 2
    recv_peer = np.concatenate([np.full(c, q, np.int32) for q, c in counts.items()])
    side = types.SimpleNamespace(npeers=npeers, me=2, recv_peer=recv_peer)
    n_tiles = -(-recv_peer.size // tile_rows)
    order = _tiles_by_peer_distance(side, n_tiles, tile_rows)
    assert sorted(order.tolist()) == list(range(n_tiles))
    peers_in_order = recv_peer[order * tile_rows].tolist()
    assert peers_in_order == [3] * 2 + [0] * 5 + [1] * 3           # 3, then round the line: 0, 1
    first = []
    for m in range(4):
        rp = np.repeat(np.array([q for q in range(4) if q != m], np.int32), 16)
        sm = types.SimpleNamespace(npeers=4, me=m, recv_peer=rp)
        first.append(int(rp[_tiles_by_peer_distance(sm, 6, 8)[0] * 8]))
    assert first == [1, 2, 3, 0]                                   # four ranks, four different first owners
    two = types.SimpleNamespace(npeers=2, me=0, recv_peer=np.ones(32, np.int32))
    assert _tiles_by_peer_distance(two, 4, 8).tolist() == [0, 1, 2, 3]
    monkeypatch.setenv("SP3_FUSED_ROTATE", "0")
    assert _tiles_by_peer_distance(side, n_tiles, tile_rows).tolist() == list(range(n_tiles))
