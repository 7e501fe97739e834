"""Host arithmetic of the L2-side-aware tile order (no GPU): the route is a permutation, each side's units
work through one contiguous part of the tile sequence sized by the side's share of the work, and every trip
of a side is a dense run. Counterpart of the route table the reference builds in
kernels/gemm/matmul/sm100.cu:635-660."""
import ctypes

import numpy as np
import pytest

from gpu_kernels_b200 import _lib


def side_route(sides, tiles):
    lib = _lib.load()
    sides = np.asarray(sides, dtype=np.uint8)
    out = (ctypes.c_uint * max(tiles, 1))()
    _lib.check(lib.gpu_kernels_nvfp4_side_route(sides.tobytes(), len(sides), tiles, out))
    return np.array(out[:tiles], dtype=np.int64)


@pytest.mark.parametrize("units,tiles,seed", [(74, 1024, 0), (74, 4096, 1), (148, 300, 2), (7, 7, 3), (5, 23, 4), (74, 150, 5)])
def test_route_is_a_permutation_and_sides_own_contiguous_parts(units, tiles, seed):
    rng = np.random.default_rng(seed)
    sides = rng.integers(0, 2, units)
    sides[0], sides[-1] = 0, 1
    route = side_route(sides, tiles)
    assert sorted(route.tolist()) == list(range(tiles))
    trips = [(tiles - 1 - u) // units + 1 if u < tiles else 0 for u in range(units)]
    work0 = sum(t for t, s in zip(trips, sides) if s == 0)
    for w, tile in enumerate(route):
        unit = w % units
        assert (tile < work0) == (sides[unit] == 0), (w, tile, work0)
    # every trip of a side covers a dense run of that side's part
    for side in (0, 1):
        members = [u for u in range(units) if sides[u] == side]
        base = 0 if side == 0 else work0
        for trip in range(max(trips[u] for u in members)):
            got = sorted(route[u + trip * units] for u in members if trip < trips[u])
            assert got == list(range(got[0], got[0] + len(got)))
            assert got[0] >= base


def test_one_sided_grid_keeps_the_sequence_order():
    route = side_route([0] * 8, 40)
    assert route.tolist() == list(range(40))


def test_bad_arguments_are_refused():
    lib = _lib.load()
    assert lib.gpu_kernels_nvfp4_side_route(None, 4, 4, None) == 1
    assert b"side_route" in lib.gpu_kernels_nvfp4_last_error()
