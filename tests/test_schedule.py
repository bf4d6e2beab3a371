"""Host-side property test of the work schedules of the persistent tensor-core GEMM kernels.

A launch of `grid` CTAs walks `total_units` work units (CTA c takes units c, c + grid, ...); `decode_unit_on`
(dfdx_b200/csrc/tc_device.cuh) turns a unit into (tile, k-block range).  Four schedules exist: K slices, stream-K,
the split of the last partial round of tiles over all CTAs, and the split for fewer tiles than CTAs.  Whatever the
schedule, every k-block of every tile must be computed exactly once -- the partial results are added into the
output -- and no CTA may get much more than its share.  The decoder is compiled for the host from the very header
the kernels include (tests/host_schedule.cu); the plan parameters are restated here from the launchers in gemm_tc.cu.
"""
import ctypes as C
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def decoder(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc not available")
    out = tmp_path_factory.mktemp("schedule") / "libhost_schedule.so"
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           f"-I{ROOT / 'include'}", str(ROOT / "tests" / "host_schedule.cu"), "-o", str(out)]
    subprocess.run(cmd, check=True, capture_output=True)
    lib = C.CDLL(str(out))
    ll, i = C.c_longlong, C.c_int
    lib.schedule_units.argtypes = [ll, i, ll, ll, i, i, i, ll, ll, i, i, i, C.POINTER(ll)]
    lib.schedule_units.restype = i

    def run(tiles, kb, grid, units, ksplit=1, kb_per_slice=None, streamk=0, sk_per_cta=0, tail_from=0, tail_per=0,
            kt_cut=0, kt_per=0):
        buf = (ll * (3 * units))()
        assert lib.schedule_units(tiles, kb, grid, units, ksplit, kb if kb_per_slice is None else kb_per_slice, streamk,
                                  sk_per_cta, tail_from, tail_per, kt_cut, kt_per, buf) == 0
        return [(buf[3 * u], buf[3 * u + 1], buf[3 * u + 2]) for u in range(units)]
    return run


def check_cover(units, tiles, kb, grid, max_share=None):
    """Every k-block of every tile exactly once; returns the k-blocks each CTA computes."""
    ranges = [[] for _ in range(tiles)]
    per_cta = [0] * grid
    for u, (tile, lo, hi) in enumerate(units):
        assert 0 <= lo <= hi <= kb
        if hi > lo:
            assert 0 <= tile < tiles
            ranges[tile].append((lo, hi))
            per_cta[u % grid] += hi - lo
    for t, r in enumerate(ranges):
        r.sort()
        assert r and r[0][0] == 0 and r[-1][1] == kb, f"tile {t}: {r}"
        assert all(r[i][1] == r[i + 1][0] for i in range(len(r) - 1)), f"tile {t}: gap or overlap in {r}"
    if max_share is not None:
        assert max(per_cta) <= max_share, (max(per_cta), max_share)
    return per_cta


def ceil_div(a, b):
    return -(-a // b)


@pytest.mark.parametrize("tiles,kb,s", [(32, 64, 4), (5, 37, 3), (1, 1024, 37), (128, 16, 2), (7, 9, 4)])
def test_k_slices(decoder, tiles, kb, s):
    kb_per = ceil_div(kb, s)
    slices = ceil_div(kb, kb_per)
    units = decoder(tiles, kb, 148, tiles * slices, ksplit=slices, kb_per_slice=kb_per)
    check_cover(units, tiles, kb, 148)


@pytest.mark.parametrize("tiles,kb,grid", [(512, 64, 148), (128, 1024, 148), (3, 1000, 148), (149, 5, 148), (300, 7, 140)])
def test_stream_k(decoder, tiles, kb, grid):
    per_cta = ceil_div(tiles * kb, grid)
    per_cta_tiles = ceil_div(per_cta, kb) + 1                       # tiles a CTA's range can touch
    units = decoder(tiles, kb, grid, grid * per_cta_tiles, streamk=1, sk_per_cta=per_cta)
    check_cover(units, tiles, kb, grid, max_share=per_cta)


@pytest.mark.parametrize("tiles,kb,grid", [(512, 64, 148), (150, 16, 148), (448, 36, 148), (512, 64, 140), (295, 300, 148),
                                           (149, 1000, 148), (2048, 64, 148)])
def test_split_of_the_last_partial_round(decoder, tiles, kb, grid):
    full, rem = divmod(tiles, grid)
    assert full >= 1 and rem > 0
    per = max(ceil_div(rem * kb, grid), 4)
    if per >= kb:
        pytest.skip("the launcher keeps whole tiles here")
    tail_from = full * grid
    units = decoder(tiles, kb, grid, tail_from + 2 * grid, tail_from=tail_from, tail_per=per)
    shares = check_cover(units, tiles, kb, grid, max_share=full * kb + per)
    assert min(shares) >= full * kb                                 # every CTA still computes its whole tiles


@pytest.mark.parametrize("tiles,kb,grid", [(128, 1024, 148), (100, 64, 148), (96, 65, 148), (128, 512, 140), (147, 4000, 148),
                                           (75, 300, 148)])
def test_fewer_tiles_than_ctas(decoder, tiles, kb, grid):
    extra = grid - tiles
    per = ceil_div(tiles, extra)
    cut = int((per * kb + 8.0 * per) / (1.0 + per)) + 1
    if cut >= kb or kb - cut < 4:
        pytest.skip("the launcher keeps whole tiles here")
    units = decoder(tiles, kb, grid, grid * per, kt_cut=cut, kt_per=per)
    shares = check_cover(units, tiles, kb, grid, max_share=max(cut, per * (kb - cut)))
    assert shares[:tiles] == [cut] * tiles                          # CTA c: k-blocks [0, cut) of tile c, all in step
    # the first unit of every CTA is its non-empty one(s): empty units only follow
    for c in range(grid):
        mine = [units[u] for u in range(c, len(units), grid)]
        seen_empty = False
        for (_, lo, hi) in mine:
            if hi == lo:
                seen_empty = True
            else:
                assert not seen_empty
