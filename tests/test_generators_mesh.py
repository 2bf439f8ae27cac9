import numpy as np
import pytest

from spcomm3d_b200.parallel.mesh import Mesh3D, dims_create, split_k, split_nnz
from spcomm3d_b200.utils import generate


def test_fixed_degree_properties_and_determinism():
    a = generate.fixed_degree(300, 200, 16, seed=4)
    b = generate.fixed_degree(300, 200, 16, seed=4)
    c = generate.fixed_degree(300, 200, 16, seed=5)
    assert (a.cols == b.cols).all() and (a.vals == b.vals).all() and not (a.cols == c.cols).all()
    cols = a.cols.reshape(300, 16)
    assert (np.diff(cols, axis=1) > 0).all()  # distinct, ascending
    assert (np.bincount(a.rows) == 16).all() and 0 <= a.vals.min() and a.vals.max() < 1
    dense = generate.fixed_degree(10, 8, 7, seed=1)  # degree close to the column count
    assert (np.diff(dense.cols.reshape(10, 7), axis=1) > 0).all()


def test_rmat_unique_sorted_skewed():
    m = generate.rmat(12, 8, seed=3)
    keys = m.rows.astype(np.int64) * m.ncols + m.cols
    assert (np.diff(keys) > 0).all() and m.nrows == 4096 and m.nnz <= 8 * 4096
    deg = np.bincount(m.rows, minlength=m.nrows)
    assert deg[: m.nrows // 2].sum() > 2 * deg[m.nrows // 2:].sum()  # a+b = 0.76 of the mass in the top half


def test_zipf_and_er_degree_laws():
    z = generate.zipf_rows(20000, 100000, alpha=1.8, dmax=4096, seed=1)
    deg = np.bincount(z.rows, minlength=20000)
    assert deg.min() >= 1 and deg.max() <= 4096 and 8 < deg.mean() < 40
    assert (deg == 1).mean() > 0.3  # heavy head at degree 1
    e = generate.erdos_renyi(20000, 20000, 32, seed=1)
    d = np.bincount(e.rows, minlength=20000)
    assert abs(d.mean() - 32) < 0.5 and abs(d.var() - 32) < 3


def test_from_spec():
    assert generate.from_spec("uniform:10:12:3", 1).nnz == 30
    assert generate.from_spec("rmat:8:4", 1).nrows == 256
    assert generate.from_spec("er:100:100:5", 1).shape == (100, 100)
    with pytest.raises(ValueError):
        generate.from_spec("nope:1")


def test_fill_rows_is_a_function_of_global_position():
    full = generate.fill_rows(np.arange(10), 16, 0, 16, seed=3, stream=1, dtype=np.float64)
    part = generate.fill_rows([7, 2], 16, 4, 8, seed=3, stream=1, dtype=np.float64)
    assert np.array_equal(part, full[[7, 2], 4:12])
    chk = generate.fill_rows([1500], 4, 0, 4, kind=generate.FILL_GID_OVER_1000, dtype=np.float64)
    assert np.allclose(chk, 1.5)


def test_dims_create_matches_mpi():
    assert dims_create(8, 2) == (2, 2, 2) and dims_create(8, 1) == (4, 2, 1) and dims_create(8, 8) == (1, 1, 8)
    assert dims_create(4, 2) == (2, 1, 2) and dims_create(4, 1) == (2, 2, 1)
    assert dims_create(2, 2) == (1, 1, 2) and dims_create(2, 1) == (2, 1, 1) and dims_create(6, 1) == (3, 2, 1)
    with pytest.raises(ValueError):
        dims_create(8, 3)


def test_rank_orders_and_fibers():
    m = Mesh3D(2, 3, 4)
    for r in range(m.size):
        assert m.rank_of(*m.coords_of(r)) == r
    assert m.rank_of(1, 2, 3) == (1 * 3 + 2) * 4 + 3  # z fastest, the MPI Cartesian order
    mx = Mesh3D(2, 3, 4, order="x_fastest")
    assert mx.rank_of(1, 2, 3) == 1 + 2 * 2 + 2 * 3 * 3  # the reference's Mesh3D helper
    r = m.rank_of(1, 1, 2)
    assert m.neighbors_z(r) == [m.rank_of(1, 1, k) for k in range(4)]
    assert len(m.neighbors_x(r)) == 2 and len(m.neighbors_y(r)) == 3 and r in m.xy_plane(r)


def test_k_and_nnz_splits():
    for k, Z in ((128, 2), (7, 2), (20, 8), (5, 8)):
        parts = [split_k(k, Z, z) for z in range(Z)]
        assert sum(w for _, w in parts) == k and parts[0][0] == 0
        assert all(o + w == parts[i + 1][0] for i, (o, w) in enumerate(parts[:-1]))
        assert [w for _, w in parts] == [k // Z + (1 if z < k % Z else 0) for z in range(Z)]
    assert split_nnz(10, 4, 1) == (3, 3) and split_nnz(10, 4, 3) == (8, 2)


def test_random_nnz_exact_count_unique_and_seeded():
    a = generate.random_nnz(300, 200, 5000, seed=4)
    b = generate.from_spec("random:300:200:5000", seed=4)
    c = generate.random_nnz(300, 200, 5000, seed=5)
    assert a.nnz == 5000 and np.all(a.vals == 1.0)
    keys = a.rows.astype(np.int64) * 200 + a.cols
    assert np.all(np.diff(keys) > 0) and a.rows.max() < 300 and a.cols.max() < 200
    assert np.array_equal(a.rows, b.rows) and np.array_equal(a.cols, b.cols)
    assert not (np.array_equal(a.rows, c.rows) and np.array_equal(a.cols, c.cols))
    full = generate.random_nnz(7, 9, 63, seed=1)
    assert full.nnz == 63
