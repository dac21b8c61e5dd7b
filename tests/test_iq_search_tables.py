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


def test_search_table_rejects_other_types():
    from libgguf_b200._native import lib
    assert lib.libgguf_cuda_iq_search_table(12, None, None, None, None, None, None, None) == 2
