"""Single-process simulators over a virtual processor mesh.

`serial_sim` counts, for every processor of an X x Y mesh, the exact sparse
send/receive messages and dense rows, and the closed-form volumes of the
sparsity-agnostic (whole-slab broadcast) method -- the job of the reference's
miniapp/serialSim.cpp:109-252, which sweeps P = 64 ... 32768.
`count_excess` is the memory-excess metric of miniapp/countExcess.cpp:135-155.
`find_xy` picks the most square X x Y (serialSim.cpp:100-106).
Both run in the native host library (csrc/host/serial_sim.cpp).
"""
from __future__ import annotations

import numpy as np

from ..utils import native
from ..utils.sparse import CooMatrix

SIM_FIELDS = ("avgSendMsgs", "avgSendVol", "avgRecvMsgs", "avgRecvVol",
              "maxSendMsgs", "maxSendVol", "maxRecvMsgs", "maxRecvVol")
MODES = {"sddmm": 0, "spmm_pre": 1, "spmm_post": 2}


def find_xy(P: int) -> tuple[int, int]:
    y = int(P ** 0.5)
    while P % y:
        y -= 1
    return P // y, y


def serial_sim(m: CooMatrix, X: int, Y: int, seed: int = 0, policy: str = "respect_comm",
               mode: str = "sddmm", dense_as_messages: bool = False) -> dict:
    """dense_as_messages: count the dense method as one message and one copy of the own block per other rank
    of the line (the reference simulator's closed form, serialSim.cpp:233-247) instead of one broadcast."""
    out = np.zeros(16, np.float64)
    rc = native.host().sp3_serial_sim(m.nnz, native.ptr(m.rows), native.ptr(m.cols), m.nrows, m.ncols, X, Y,
                                      seed, {"respect_comm": 0, "random": 1}[policy],
                                      MODES[mode] + (16 if dense_as_messages else 0), native.ptr(out))
    native.check(rc, "serial_sim")
    return {"sparse": dict(zip(SIM_FIELDS, out[:8].tolist())), "dense": dict(zip(SIM_FIELDS, out[8:].tolist()))}


def sim_line(tag: str, m: CooMatrix, P: int, stats: dict) -> str:
    """One report line: `<tag S|B> <matrix> <P> <nnz> <8 fields>` (the S / B
    lines of serialSim.cpp:227-230,249-252)."""
    return f"{tag} {m.name} {P} {m.nnz} " + " ".join(f"{stats[f]:.2f}" for f in SIM_FIELDS)


def find_xy_ref(P: int) -> tuple[int, int]:
    """X x Y as the reference's simulator picks it: X the largest divisor of P not above sqrt(P), Y = P / X
    (serialSim.cpp:100-106)."""
    y, x = find_xy(P)
    return x, y


def sim_line_ref(tag: str, m: CooMatrix, N: int, X: int, Y: int, Z: int, f: int, stats: dict) -> str:
    """The line the reference's simulator prints (serialSim.cpp:227-230, 249-252):
    `name rows cols nnz N XxYxZ f c S|B avgSendMsgs avgSendVol avgRecvMsgs avgRecvVol maxSendMsgs maxSendVol
    maxRecvMsgs maxRecvVol`, averages with two decimals, maxima as integers, volumes in dense rows."""
    avg = " ".join(f"{stats[k]:.2f}" for k in SIM_FIELDS[:4])
    mx = " ".join(str(int(round(stats[k]))) for k in SIM_FIELDS[4:])
    return f"{m.name} {m.nrows} {m.ncols} {m.nnz} {N} {X}x{Y}x{Z} {f} {Z} {tag} {avg} {mx}"


def count_excess(m: CooMatrix, X: int, Y: int, seed: int = 0) -> dict:
    out = np.zeros(3, np.float64)
    rc = native.host().sp3_count_excess(m.nnz, native.ptr(m.rows), native.ptr(m.cols), m.nrows, m.ncols, X, Y,
                                        seed, native.ptr(out))
    native.check(rc, "count_excess")
    return {"stored_rows": out[0], "touched_rows": out[1], "excess_rows": out[2]}


def count_empty(m: CooMatrix) -> tuple[int, int]:
    """(rows, columns) without any nonzero (tools/countEmptyRows.cpp:80-92)."""
    import ctypes
    er, ec = ctypes.c_uint64(), ctypes.c_uint64()
    rc = native.host().sp3_count_empty(m.nnz, native.ptr(m.rows), native.ptr(m.cols), m.nrows, m.ncols,
                                       ctypes.addressof(er), ctypes.addressof(ec))
    native.check(rc, "count_empty")
    return er.value, ec.value
