"""How the embedding-layer GEMMs deal their work to the CTAs (host logic of the engine, no GPU): equal shares, every
column of every (M tile, K split) exactly once, units within the accumulator width, staggered first units."""
import ctypes as C

import numpy as np
import pytest

from multigputrainmlp_b200 import _lib


def work_list(grid, m_tiles, splits, n_begin, n_end, max_cols=512):
    lib = _lib.load()
    lib.mgt_debug_work_list.argtypes = [C.c_uint32] * 6 + [C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32)]
    cap = grid * 128
    out = np.zeros((cap, 4), np.uint32)
    stride = C.c_uint32(0)
    st = lib.mgt_debug_work_list(grid, m_tiles, splits, n_begin, n_end, max_cols, out.ctypes.data_as(C.c_void_p), cap, C.byref(stride))
    if st != 0:
        return st, None
    units = out[: grid * stride.value].reshape(grid, stride.value, 4)
    per_cta = []
    for b in range(grid):
        mine = []
        for mt, n_base, n_count, sp in units[b]:
            if n_count == 0:
                break
            mine.append((int(mt), int(n_base), int(n_count), int(sp)))
        assert len(mine) < stride.value  # the terminator fits
        per_cta.append(mine)
    return 0, per_cta


@pytest.mark.parametrize("grid,m_tiles,splits,n_begin,n_end", [
    (148, 20, 1, 0, 53248),        # embedding forward at p888: 2560 columns x 53 248 samples
    (148, 20, 2, 0, 2592),         # embedding gradient, first block of 36 positions
    (148, 20, 2, 2592, 5184),      # ... second block
    (148, 20, 2, 0, 5184),         # all rows in one launch
    (148, 32, 1, 0, 131072),       # hd1 4096, batch 131 072
    (7, 1, 1, 0, 300), (3, 2, 2, 10, 77), (148, 1, 1, 0, 96), (40, 5, 2, 0, 1000),
])
def test_every_column_once_and_equal_shares(grid, m_tiles, splits, n_begin, n_end):
    st, per_cta = work_list(grid, m_tiles, splits, n_begin, n_end)
    assert st == 0
    seen = np.zeros((m_tiles, splits, n_end - n_begin), np.int32)
    totals = []
    for mine in per_cta:
        totals.append(sum(u[2] for u in mine))
        for mt, n_base, n_count, sp in mine:
            assert 0 < n_count <= 512 and n_begin <= n_base and n_base + n_count <= n_end and mt < m_tiles and sp < splits
            seen[mt, sp, n_base - n_begin:n_base - n_begin + n_count] += 1
    assert (seen == 1).all()
    busy = [t for t in totals if t > 0]
    share = -(-m_tiles * splits * (n_end - n_begin) // grid)
    assert max(busy) <= (share + 15) // 16 * 16            # nobody has more than an equal share (rounded up to 16 columns)
    assert sum(1 for t in totals if t < max(busy)) <= 1 + (grid - len(busy))  # only the last busy CTA may have less


def test_first_units_are_staggered_at_p888():
    st, per_cta = work_list(148, 20, 1, 0, 53248)
    firsts = [mine[0][2] for mine in per_cta]
    assert len(set(firsts)) >= 8                            # CTAs reach their first epilogue at different times
    assert all(len(mine) <= 17 for mine in per_cta)         # 7200 columns each: 15 units of <= 512, plus an M-tile crossing
    # whole tiles dealt round-robin would give 2080 / 148 = 14.05 -> 15 rounds of 512; equal shares are 7200 columns
    assert max(sum(u[2] for u in mine) for mine in per_cta) == 7200


def test_invalid_requests():
    assert work_list(0, 20, 1, 0, 100)[0] == 1
    assert work_list(148, 20, 1, 5, 5)[0] == 1
    assert work_list(1, 64, 2, 0, 53248)[0] == 1             # one CTA cannot hold that many units: no list, tiles are dealt instead
