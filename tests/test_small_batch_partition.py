"""Host arithmetic of the small-batch kernel's work partition (no GPU): every work unit belongs to
exactly one CTA, the ranges are contiguous, ordered and differ by at most one unit in length, and
the closed-form owner agrees with the ranges — for the shapes the kernel meets and for awkward
unit / CTA counts."""
import ctypes

import pytest


def _partition(lib, units, ctas):
    begins = []
    b, e = ctypes.c_longlong(0), ctypes.c_longlong(0)
    for c in range(ctas):
        assert lib.mlxr_debug_smallm_partition(units, ctas, c, 0, ctypes.byref(b), ctypes.byref(e), None) == 0
        begins.append((b.value, e.value))
    return begins


@pytest.mark.parametrize("units,ctas", [(1, 1), (5, 5), (7, 3), (148, 148), (149, 148), (1792, 148), (3584, 148),
                                        (224 * 16, 132), (32 * 56, 148), (1000003, 148), (2 ** 33, 148)])
def test_ranges_cover_every_unit_once(units, ctas):
    from mlxr_b200._capi import lib
    r = _partition(lib, units, ctas)
    assert r[0][0] == 0 and r[-1][1] == units
    for (b0, e0), (b1, _) in zip(r, r[1:]):
        assert e0 == b1
    sizes = [e - b for b, e in r]
    assert min(sizes) >= 1 and max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("units,ctas", [(7, 3), (149, 148), (1792, 148), (3584, 148), (32 * 56, 148), (997, 31)])
def test_owner_matches_ranges(units, ctas):
    from mlxr_b200._capi import lib
    r = _partition(lib, units, ctas)
    o = ctypes.c_int(-1)
    probes = set()
    for c, (b, e) in enumerate(r):
        probes.update({(b, c), (e - 1, c)})
    probes.update((u, None) for u in range(0, units, max(1, units // 97)))
    for u, want in probes:
        assert lib.mlxr_debug_smallm_partition(units, ctas, 0, u, None, None, ctypes.byref(o)) == 0
        b, e = r[o.value]
        assert b <= u < e
        if want is not None:
            assert o.value == want


def test_contributors_per_tile():
    """Tiles of nsb units each: the number of CTAs sharing tile t is owner(last unit) - owner(first
    unit) + 1, and the sum over tiles of (contributors - 1) is the number of ranges that cross a
    tile boundary."""
    from mlxr_b200._capi import lib
    ntiles, nsb, ctas = 112, 16, 148
    units = ntiles * nsb
    r = _partition(lib, units, ctas)
    o0, o1 = ctypes.c_int(0), ctypes.c_int(0)
    shared = 0
    for t in range(ntiles):
        lib.mlxr_debug_smallm_partition(units, ctas, 0, t * nsb, None, None, ctypes.byref(o0))
        lib.mlxr_debug_smallm_partition(units, ctas, 0, (t + 1) * nsb - 1, None, None, ctypes.byref(o1))
        nc = o1.value - o0.value + 1
        assert 1 <= nc <= 3
        assert nc == sum(1 for b, e in r if b < (t + 1) * nsb and e > t * nsb)
        shared += nc - 1
    crossing = sum(1 for b, e in r if b // nsb != (e - 1) // nsb)
    assert shared >= crossing


def test_rejects_bad_arguments():
    from mlxr_b200._capi import lib
    assert lib.mlxr_debug_smallm_partition(10, 11, 0, 0, None, None, None) != 0
    assert lib.mlxr_debug_smallm_partition(10, 5, 5, 0, None, None, None) != 0
    assert lib.mlxr_debug_smallm_partition(10, 5, 0, 10, None, None, None) != 0
