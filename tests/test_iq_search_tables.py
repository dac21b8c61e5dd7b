"""The lattice quantizers' search tables (grid, lattice-point map, neighbour lists) against the ones the upstream
library builds for itself (csrc/common/libgguf_iq_tables.cpp:36-417 iq2xs_init_impl -> iq2_data[4],
:487-666 iq3xs_init_impl -> iq3_data[2]).  Host only: both sides are built on the CPU.  The quantizers keep the
first strict minimum over a neighbour list, so the order of every list is part of the encoded result."""
import ctypes

import numpy as np
import pytest


class _Entry(ctypes.Structure):
    _fields_ = [("grid", ctypes.c_void_p), ("map", ctypes.c_void_p), ("neighbours", ctypes.c_void_p)]


# qtype -> (upstream table array, index in it, argument of its init function, grid size, coordinates, map size)
CASES = {
    "IQ2_XXS": (16, "iq2", 0, 16, 256, 8, 43692),
    "IQ2_XS": (17, "iq2", 1, 17, 512, 8, 43692),
    "IQ1_S": (19, "iq2", 2, 19, 2048, 8, 43692),
    "IQ1_M": (29, "iq2", 2, 29, 2048, 8, 43692),
    "IQ2_S": (22, "iq2", 3, 22, 1024, 8, 43692),
    "IQ3_XXS": (18, "iq3", 0, 256, 256, 4, 4096),
    "IQ3_S": (21, "iq3", 1, 512, 512, 4, 4096),
}


def _ours(qtype):
    from libgguf_b200._native import lib
    gs, dims = ctypes.c_int32(), ctypes.c_int32()
    grid, mp, nb = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
    msize, nlen = ctypes.c_int64(), ctypes.c_int64()
    assert lib.libgguf_cuda_iq_search_table(qtype, ctypes.byref(gs), ctypes.byref(dims), ctypes.byref(grid), ctypes.byref(mp),
                                            ctypes.byref(msize), ctypes.byref(nb), ctypes.byref(nlen)) == 0
    g = np.ctypeslib.as_array(ctypes.cast(grid.value, ctypes.POINTER(ctypes.c_uint8)), (gs.value * dims.value,)).reshape(gs.value, dims.value)
    m = np.ctypeslib.as_array(ctypes.cast(mp.value, ctypes.POINTER(ctypes.c_int32)), (msize.value,))
    n = np.ctypeslib.as_array(ctypes.cast(nb.value, ctypes.POINTER(ctypes.c_uint16)), (nlen.value,))
    return g, m, n


@pytest.mark.parametrize("name", sorted(CASES))
def test_search_tables_equal_upstreams(ref, name):
    qtype, family, index, init_arg, grid_size, dims, map_size = CASES[name]
    up = ref.lib
    if family == "iq2":
        up.iq2xs_init_impl(ctypes.c_int(init_arg))
        entry = (_Entry * 4).in_dll(up, "iq2_data")[index]
    else:
        up.iq3xs_init_impl(ctypes.c_int(init_arg))
        entry = (_Entry * 2).in_dll(up, "iq3_data")[index]
    assert entry.grid and entry.map and entry.neighbours
    grid, mp, nb = _ours(qtype)
    assert grid.shape == (grid_size, dims) and mp.shape == (map_size,)
    # grid: upstream packs the coordinates of an entry into one little-endian word (8 or 4 bytes)
    up_grid = np.ctypeslib.as_array(ctypes.cast(entry.grid, ctypes.POINTER(ctypes.c_uint8)), (grid_size * dims,)).reshape(grid_size, dims)
    np.testing.assert_array_equal(grid, up_grid)
    up_map = np.ctypeslib.as_array(ctypes.cast(entry.map, ctypes.POINTER(ctypes.c_int32)), (map_size,))
    np.testing.assert_array_equal(mp, up_map)
    # the neighbour array's length is implied by the map: the last list's offset + 1 + its count
    off_last = int((-mp[mp < 0] - 1).max())
    up_nb_head = np.ctypeslib.as_array(ctypes.cast(entry.neighbours, ctypes.POINTER(ctypes.c_uint16)), (off_last + 1,))
    total = off_last + 1 + int(up_nb_head[off_last])
    assert total == nb.shape[0]
    up_nb = np.ctypeslib.as_array(ctypes.cast(entry.neighbours, ctypes.POINTER(ctypes.c_uint16)), (total,))
    np.testing.assert_array_equal(nb, up_nb)
    # every point that is not on the grid has a non-empty list
    offs = -mp[mp < 0] - 1
    assert (nb[offs] > 0).all()


@pytest.mark.parametrize("name", ["IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ1_S", "IQ1_M"])
def test_scan_records_hold_upstreams_lists(name):
    """The layout the IQ2 / IQ3 kernels scan is derived from the lists above: same entries in the same order, a tail of
    copies of the first entry up to a whole record, records back to back, map_s pointing at them."""
    from libgguf_b200._native import lib
    qtype, _, _, _, grid_size, dims, map_size = CASES[name]
    _, mp, nb = _ours(qtype)
    per, n_entries, n_map = ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int64()
    ent, ms = ctypes.c_void_p(), ctypes.c_void_p()
    assert lib.libgguf_cuda_iq_scan_records(qtype, ctypes.byref(per), ctypes.byref(ent), ctypes.byref(n_entries), ctypes.byref(ms),
                                            ctypes.byref(n_map)) == 0
    per = per.value
    assert per == (8 if name == "IQ2_XS" else 4) and n_map.value == map_size and n_entries.value % per == 0
    entries = np.ctypeslib.as_array(ctypes.cast(ent.value, ctypes.POINTER(ctypes.c_uint16)), (n_entries.value,))
    map_s = np.ctypeslib.as_array(ctypes.cast(ms.value, ctypes.POINTER(ctypes.c_int32)), (map_size,))
    on_grid = mp >= 0
    np.testing.assert_array_equal(map_s[on_grid], mp[on_grid])
    assert (map_s[~on_grid] < 0).all()
    packed = (-map_s[~on_grid].astype(np.int64) - 1)
    first, count = packed >> 8, packed & 255
    offs = -mp[~on_grid].astype(np.int64) - 1
    n = nb[offs].astype(np.int64)
    np.testing.assert_array_equal(count, (n + per - 1) // per)
    # every list has a range of its own and together they tile the array (up to a tail that rounds it to 16 bytes).
    # IQ2 (a kernel keeps only the front of the array in shared memory): most common lattice point first, by the sum of
    # the point's levels (a 2-bit field of 3 is no level), then by index.  IQ3 (all of it fits): by index.
    by_start = np.argsort(first)
    np.testing.assert_array_equal(first[by_start], np.concatenate(([0], np.cumsum(count[by_start])[:-1])))
    used = int((first[by_start[-1]] + count[by_start[-1]]) * per)
    assert used <= n_entries.value < used + 8 and n_entries.value % 8 == 0
    points = np.flatnonzero(~on_grid)
    bits = 2 if dims == 8 else 3
    fields = (points[:, None] >> (bits * np.arange(dims))) & ((1 << bits) - 1)
    key = np.where((bits == 2) & (fields == 3), 1000, fields).sum(1) if dims == 8 else np.zeros(len(points), np.int64)
    assert (np.diff(key[by_start]) >= 0).all()
    same = np.diff(key[by_start]) == 0
    assert (np.diff(points[by_start])[same] > 0).all()
    assert int(entries.max()) == (grid_size - 1) * dims * 2 or int(entries.max()) < grid_size * dims * 2
    for i in np.random.default_rng(0).choice(len(offs), 400, replace=False).tolist() + [0, len(offs) - 1, int(np.argmax(n))]:
        want = nb[offs[i] + 1:offs[i] + 1 + n[i]].astype(np.int64) * dims * 2
        got = entries[first[i] * per:(first[i] + count[i]) * per].astype(np.int64)
        np.testing.assert_array_equal(got[:n[i]], want)
        assert (got[n[i]:] == want[0]).all()


def test_scan_records_reject_other_types():
    from libgguf_b200._native import lib
    assert lib.libgguf_cuda_iq_scan_records(12, None, None, None, None, None) == 2
    assert lib.libgguf_cuda_iq_scan_records(20, None, None, None, None, None) == 2   # IQ4_NL has no lattice search


def test_search_table_rejects_other_types():
    from libgguf_b200._native import lib
    assert lib.libgguf_cuda_iq_search_table(12, None, None, None, None, None, None, None) == 2
