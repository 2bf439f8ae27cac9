"""conv2bin binary format, MatrixMarket quirks, native conv2bin tool."""
import struct
import subprocess

import numpy as np
import pytest

from spcomm3d_b200.utils import binfmt, generate, native
from spcomm3d_b200.utils.sparse import CooMatrix


def test_bin_layout_and_roundtrip(tmp_path):
    m = CooMatrix(3, 4, [0, 2, 1], [3, 0, 1], [1.5, -2.0, 3.25])
    p = str(tmp_path / "t.bin")
    binfmt.write_bin(p, m)
    raw = open(p, "rb").read()
    assert len(raw) == 16 + 3 * 16
    assert struct.unpack("<IIQ", raw[:16]) == (3, 4, 3)
    assert struct.unpack("<IId", raw[16:32]) == (0, 3, 1.5)
    assert struct.unpack("<IId", raw[32:48]) == (2, 0, -2.0)
    back = binfmt.read_bin(p)
    assert back.shape == (3, 4) and back.name == "t"
    assert (back.rows == m.rows).all() and (back.cols == m.cols).all() and (back.vals == m.vals).all()
    part = binfmt.read_bin(p, 1, 2)
    assert part.rows.tolist() == [2, 1]


def test_chunk_ranges_cover_file():
    for nnz in (0, 1, 7, 100):
        for parts in (1, 3, 8):
            spans = [binfmt.chunk_range(nnz, parts, i) for i in range(parts)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == nnz
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1


def test_truncated_and_out_of_range_files(tmp_path):
    p = str(tmp_path / "bad.bin")
    with open(p, "wb") as f:
        f.write(struct.pack("<IIQ", 2, 2, 5))
        f.write(struct.pack("<IId", 0, 0, 1.0))
    with pytest.raises(native.NativeError):
        binfmt.read_bin_header(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<IIQ", 2, 2, 1))
        f.write(struct.pack("<IId", 5, 0, 1.0))
    with pytest.raises(native.NativeError):
        binfmt.read_bin(p)


MTX_GENERAL = """%%MatrixMarket matrix coordinate real general
% a comment
%another
3 4 3
1 4 1.5
3 1 -2
2 2 3.25
"""
MTX_SYMM = """%%MatrixMarket matrix coordinate real symmetric
3 3 3
1 1 4.0
2 1 1.0
3 2 2.0
"""
MTX_PATTERN = """%%MatrixMarket matrix coordinate pattern general
2 2 2
1 2
2 1
"""
MTX_COMPLEX = """%%MatrixMarket matrix coordinate complex general
2 2 1
2 2 1.5 -7.0
"""


def _write(tmp_path, name, text):
    p = tmp_path / name
    p.write_text(text)
    return str(p)


def test_mtx_general(tmp_path):
    m = binfmt.read_mtx(_write(tmp_path, "g.mtx", MTX_GENERAL))
    assert m.shape == (3, 4) and m.rows.tolist() == [0, 2, 1] and m.cols.tolist() == [3, 0, 1]
    assert m.vals.tolist() == [1.5, -2.0, 3.25]


def test_mtx_symmetric_mirrors_everything_like_the_reference(tmp_path):
    p = _write(tmp_path, "s.mtx", MTX_SYMM)
    m = binfmt.read_mtx(p)
    # second half holds the mirrored entries in file order, diagonal included
    assert m.nnz == 6
    assert m.rows.tolist() == [0, 1, 2, 0, 0, 1] and m.cols.tolist() == [0, 0, 1, 0, 1, 2]
    d = binfmt.read_mtx(p, mirror_diagonal=False)
    assert d.nnz == 5 and d.rows.tolist() == [0, 1, 2, 0, 1]


def test_mtx_pattern_and_complex(tmp_path):
    m = binfmt.read_mtx(_write(tmp_path, "p.mtx", MTX_PATTERN))
    assert m.vals.tolist() == [1.0, 1.0]
    c = binfmt.read_mtx(_write(tmp_path, "c.mtx", MTX_COMPLEX))
    assert c.vals.tolist() == [1.5] and c.rows.tolist() == [1]


def test_native_conv2bin_matches_python(tmp_path):
    exe = native.build_tools()
    p = _write(tmp_path, "s.mtx", MTX_SYMM)
    out = subprocess.run([str(exe), p], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    native_bytes = open(str(tmp_path / "s.bin"), "rb").read()
    py = binfmt.conv2bin(p, str(tmp_path / "py.bin"))
    assert native_bytes == open(py, "rb").read()
    assert subprocess.run([str(exe)], capture_output=True).returncode == 2


def test_mtx_write_read_roundtrip(tmp_path):
    m = generate.fixed_degree(50, 40, 3, seed=2)
    p = str(tmp_path / "w.mtx")
    binfmt.write_mtx(p, m)
    b = binfmt.read_mtx(p)
    assert (b.rows == m.rows).all() and (b.cols == m.cols).all() and np.allclose(b.vals, m.vals)
