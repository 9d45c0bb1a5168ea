"""CPU tests of the attention launcher's work planning (rfk_flash_attention_plan, host only): which grids are cut
along the keys, and that a cut covers every key tile of every unit exactly once with consistent slot bookkeeping."""
import ctypes

import pytest

import renderformer_cuda_b200 as pkg  # noqa: F401
from renderformer_cuda_b200 import _abi


def _plan(units, n_tiles, sms=148):
    lib = _abi.load("rfk.h")
    whole, n = ctypes.c_int(-1), ctypes.c_int(-1)
    buf = (ctypes.c_ushort * (6 * 320))()
    rc = lib.rfk_flash_attention_plan(units, n_tiles, sms, ctypes.byref(whole), ctypes.byref(n), ctypes.cast(buf, ctypes.c_void_p), 320)
    assert rc == 0
    pieces = [tuple(buf[6 * i + k] for k in range(6)) for i in range(n.value)]
    return whole.value, pieces


@pytest.mark.parametrize("units,n_tiles,sms", [(64, 89, 148), (12, 32, 148), (1, 64, 148), (7, 500, 132), (100, 200, 148),
                                               (3, 9, 148), (147, 1000, 148), (40, 89, 16)])
def test_cut_grids_cover_every_tile_once(units, n_tiles, sms):
    whole, pieces = _plan(units, n_tiles, sms)
    if not pieces:
        assert whole == units
        return
    assert whole == 0 and units < sms                                   # only grids that leave SMs idle are cut
    assert len(pieces) <= 320 and len(pieces) <= 2 * min(sms, 160)
    covered = {u: [0] * n_tiles for u in range(units)}
    by_unit = {}
    for unit, t0, nt, first, count, slot in pieces:
        assert nt >= 1 and t0 + nt <= n_tiles
        for t in range(t0, t0 + nt):
            covered[unit][t] += 1
        by_unit.setdefault(unit, []).append((first, count, slot))
    assert all(c == 1 for u in covered.values() for c in u), "a key tile is missed or taken twice"
    slots = sorted(s for v in by_unit.values() for _, _, s in v)
    assert slots == list(range(len(pieces)))                            # one workspace slot per piece
    for unit, recs in by_unit.items():
        first, count = recs[0][0], recs[0][1]
        assert all(r[0] == first and r[1] == count for r in recs) and count == len(recs) and count <= 9
        assert sorted(r[2] for r in recs) == list(range(first, first + count))   # the unit's slots are consecutive
    sizes = [p[2] for p in pieces]
    assert sizes == sorted(sizes, reverse=True)                         # longest first
    share = -(-units * n_tiles // min(sms, 160, units * 8))
    assert max(sizes) <= share


@pytest.mark.parametrize("units,n_tiles", [(256, 89), (148, 89), (108, 25), (4, 1), (64, 10), (300, 40), (0, 5)])
def test_grids_left_whole(units, n_tiles):
    """A grid of one round or more, or pieces so short that their fixed cost (about twelve tile times) eats the gain."""
    whole, pieces = _plan(units, n_tiles)
    assert whole == units and pieces == []


def test_plan_rejects_bad_arguments():
    lib = _abi.load("rfk.h")
    w, n = ctypes.c_int(), ctypes.c_int()
    assert lib.rfk_flash_attention_plan(4, 0, 148, ctypes.byref(w), ctypes.byref(n), None, 0) == -1
    assert lib.rfk_flash_attention_plan(4, 8, 0, ctypes.byref(w), ctypes.byref(n), None, 0) == -1
    assert lib.rfk_flash_attention_plan(4, 8, 148, None, ctypes.byref(n), None, 0) == -1
    assert lib.rfk_flash_attention_plan(64, 89, 148, ctypes.byref(w), ctypes.byref(n), None, 0) == 0 and n.value > 0   # count only
