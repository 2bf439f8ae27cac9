"""Host-side logic of the dense-panel split (ops/panel.py), no GPU: every
nonzero lands in exactly one place, panel entries agree with the panel tables,
groups respect row blocks and the cap on groups per block."""
import numpy as np
import pytest

from spcomm3d_b200.ops.panel import PANEL_M, PANEL_N, PanelSpMM


def _matrix(seed, hub_rows=300, hub_cols=200, nrows=700, ncols=600, fill=0.3, noise=3000):
    rng = np.random.default_rng(seed)
    hub = rng.choice(ncols, hub_cols, replace=False)
    rr, cc = np.nonzero(rng.random((hub_rows, hub_cols)) < fill)
    rows = np.concatenate([rr, rng.integers(0, nrows, noise)])
    cols = np.concatenate([hub[cc], rng.integers(0, ncols, noise)])
    keys = np.unique(rows.astype(np.int64) * ncols + cols)
    return (keys // ncols).astype(np.int32), (keys % ncols).astype(np.int32), rng.random(keys.size), nrows, ncols


@pytest.mark.parametrize("group_panels", [1, 2, 8])
def test_split_covers_every_nonzero_once(group_panels):
    rows, cols, vals, nrows, ncols = _matrix(1)
    op = PanelSpMM(rows, cols, vals, nrows, ncols, device="cpu", group_panels=group_panels)
    s = op.split
    assert op.npanels > 0 and op.n_panel_nnz + op.n_rest == rows.size
    pos = np.concatenate([s.e_pos.numpy(), s.r_pos.numpy()])
    assert np.array_equal(np.sort(pos), np.arange(rows.size))
    # panel entries: row inside the panel's block, column = the panel's column slot
    ptr = s.panel_ptr.numpy()
    panel_of = np.repeat(np.arange(op.npanels), np.diff(ptr))
    e_pos = s.e_pos.numpy()
    row0 = s.panel_row0.numpy()[panel_of]
    assert np.array_equal(rows[e_pos], row0 + s.e_row.numpy())
    assert np.all(s.e_row.numpy() < PANEL_M) and np.all(s.e_col.numpy() < PANEL_N)
    assert np.array_equal(cols[e_pos], s.panel_cols.numpy()[panel_of, s.e_col.numpy()])
    assert np.allclose(vals[e_pos], s.e_sval.numpy(), rtol=1e-6)
    # remainder: row-sorted CSR over all rows
    rp = op.rowptr.numpy()
    assert rp[-1] == op.n_rest and np.array_equal(np.diff(rp), np.bincount(s.r_row.numpy(), minlength=nrows))
    # groups: consecutive panels of one row block; shared flag iff the block has several groups
    g = op.grp_ptr.numpy()
    assert g[0] == 0 and g[-1] == op.npanels and np.all(np.diff(g) > 0)
    blocks = {}
    for i in range(op.ngroups):
        r0 = set(s.panel_row0.numpy()[g[i]:g[i + 1]].tolist())
        assert len(r0) == 1
        blocks.setdefault(r0.pop(), []).append(i)
    shared = op.grp_shared.numpy()
    for members in blocks.values():
        assert len(members) <= 16 or group_panels >= len(members)
        for i in members:
            assert bool(shared[i]) == (len(members) > 1)


def test_groups_per_block_are_capped():
    # one block with 40 column tiles: groups of ceil(40 / 16) = 3 panels, 14 groups
    rows, cols, vals, nrows, ncols = _matrix(2, hub_rows=128, hub_cols=40 * PANEL_N, nrows=256, ncols=4000,
                                             fill=0.2, noise=10)
    op = PanelSpMM(rows, cols, vals, nrows, ncols, device="cpu", group_panels=1)
    r0 = op.split.panel_row0.numpy()[:op.npanels]
    in_block0 = int((r0 == 0).sum())
    assert in_block0 >= 38
    g = op.grp_ptr.numpy()
    groups_block0 = sum(1 for i in range(op.ngroups) if r0[g[i]] == 0)
    assert groups_block0 <= 16 and int(np.diff(g).max()) == -(-in_block0 // 16)


def test_dense_reconstruction_matches():
    rows, cols, vals, nrows, ncols = _matrix(3)
    op = PanelSpMM(rows, cols, vals, nrows, ncols, device="cpu")
    s = op.split
    dense = np.zeros((nrows, ncols))
    ptr = s.panel_ptr.numpy()
    for p in range(op.npanels):
        e = slice(ptr[p], ptr[p + 1])
        r = s.panel_row0.numpy()[p] + s.e_row.numpy()[e].astype(np.int64)
        c = s.panel_cols.numpy()[p, s.e_col.numpy()[e].astype(np.int64)]
        dense[r, c] += s.e_sval.numpy()[e]
    dense[s.r_row.numpy(), s.r_col.numpy()] += s.r_val.numpy()
    ref = np.zeros((nrows, ncols))
    ref[rows, cols] = vals
    assert np.allclose(dense, ref, rtol=1e-6, atol=1e-7)
