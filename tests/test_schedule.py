"""The tile schedule of the persistent kernel, computed on the CPU by the kernel's own scheduling functions
(apk_debug_schedule): every tile exactly once, the local rank's rows first (all-gather) or behind the
peers' (reduce-scatter), peers interleaved per row block, pairs on vertically adjacent tiles."""
import ctypes as C
import itertools

import numpy as np
import pytest

from autoparallel_b200 import _native as nat
from autoparallel_b200.build import build_native

PLAIN, AG, RS = 0, 1, 2


def schedule(mode, world, rank, rows, Ns, last_dim=0, pair=0, crank=0):
    build_native()
    L = nat.lib()
    arr = (C.c_int32 * len(Ns))(*Ns)
    total = L.apk_debug_schedule(mode, world, rank, rows, len(Ns), arr, last_dim, pair, crank, None, 0)
    assert total >= 0, L.apk_last_error()
    out = np.zeros((total, 6), dtype=np.int32)
    got = L.apk_debug_schedule(mode, world, rank, rows, len(Ns), arr, last_dim, pair, crank,
                               out.ctypes.data_as(C.POINTER(C.c_int32)), total)
    assert got == total
    return out


def expected_tiles(world, rows, Ns, bn, chunks):
    mt = -(-rows // 128)
    return {(c, m, b, n0) for c in chunks for m in range(mt) for b, N in enumerate(Ns) for n0 in range(0, N, bn)}


@pytest.mark.parametrize("world,rank", [(1, 0), (2, 1), (4, 3), (8, 5)])
@pytest.mark.parametrize("rows,Ns", [(4096, [1792, 1792]), (1000, [264, 128]), (130, [8]), (512, [512, 128, 128])])
def test_all_gather_order(world, rank, rows, Ns):
    bn = 128 if max(Ns) <= 128 else 256
    s = schedule(AG, world, rank, rows, Ns)
    tiles = [tuple(r[:4]) for r in s]
    assert len(set(tiles)) == len(tiles) and set(tiles) == expected_tiles(world, rows, Ns, bn, range(world))
    per_chunk = len(tiles) // world
    assert all(t[0] == rank for t in tiles[:per_chunk])                  # own shard first: no waiting at t = 0
    nt = per_chunk // (-(-rows // 128))
    rest = tiles[per_chunk:]
    for i in range(0, len(rest), nt * max(world - 1, 1)):                # then row block by row block, peers rank+1, rank+2, ...
        block = rest[i:i + nt * (world - 1)]
        assert len({t[1] for t in block}) == 1
        assert [t[0] for t in block[::nt]] == [(rank + 1 + k) % world for k in range(world - 1)]
    assert all(r[4] == r[1] * nt + i % nt for i, r in enumerate(s))      # tile index inside the chunk
    assert s[:, 5].min() == (rows - 1) % 128 + 1 if rows % 128 else s[:, 5].min() == 128


@pytest.mark.parametrize("world,rank", [(2, 0), (4, 2), (8, 7)])
@pytest.mark.parametrize("rows,N", [(4096, 4096), (300, 264), (128, 64), (1100, 512)])
def test_reduce_scatter_order(world, rank, rows, N):
    bn = 128 if N <= 128 else 256
    s = schedule(RS, world, rank, rows, [N])
    tiles = [tuple(r[:4]) for r in s]
    assert len(set(tiles)) == len(tiles) and set(tiles) == expected_tiles(world, rows, [N], bn, range(world))
    pos = {t: i for i, t in enumerate(tiles)}
    mt = -(-rows // 128)
    lag = min(4, mt)
    for m, n0 in itertools.product(range(mt), range(0, N, bn)):
        own = pos[(rank, m, 0, n0)]
        # an own tile comes after every peer's tiles of the row block `lag` further down (or of the last one)
        ahead = min(m + lag - 1, mt - 1)
        assert all(own > pos[(c, ahead, 0, k)] for c in range(world) if c != rank for k in range(0, N, bn))
    assert tiles[-1][0] == rank


@pytest.mark.parametrize("mode,world,rank", [(PLAIN, 1, 0), (AG, 8, 3), (RS, 4, 1)])
def test_pairs_take_vertically_adjacent_tiles(mode, world, rank):
    rows, Ns = 1024, [512, 256] if mode != RS else [512]
    a = schedule(mode, world, rank, rows, Ns, pair=1, crank=0)
    b = schedule(mode, world, rank, rows, Ns, pair=1, crank=1)
    assert a.shape == b.shape
    assert (a[:, [0, 2, 3]] == b[:, [0, 2, 3]]).all() and (a[:, 1] % 2 == 0).all() and (b[:, 1] == a[:, 1] + 1).all()
    single = schedule(mode, world, rank, rows, Ns)
    both = {tuple(r[:4]) for r in a} | {tuple(r[:4]) for r in b}
    assert both == {tuple(r[:4]) for r in single} and len(both) == 2 * len(a)


def test_last_dim_variants():
    # K-split all-gather: one pass over the shard's rows, whatever the group size
    s = schedule(AG, 8, 2, 640, [512], last_dim=1)
    assert len(s) == 5 * 2 and (s[:, 0] == 0).all()
    # column-split reduce-scatter: chunks are column ranges of ALL rows
    s = schedule(RS, 4, 1, 640, [256], last_dim=1)
    assert len(s) == 4 * 5 * 1 and set(s[:, 0]) == {0, 1, 2, 3}


# ------------------------------------------------------------------------------------------------
# Properties over random shapes (the fixed cases above pin the exact order; these guard the
# invariants the device protocol relies on for every shape the host code can pass down).
# ------------------------------------------------------------------------------------------------
from hypothesis import given, settings, strategies as st  # noqa: E402


def _widths(draw, pair):
    n = draw(st.integers(1, 3))
    if pair:
        return [256 * draw(st.integers(1, 4)) for _ in range(n)]
    return [8 * draw(st.integers(1, 130)) for _ in range(n)]


@st.composite
def _shapes(draw, modes=(PLAIN, AG, RS)):
    mode = draw(st.sampled_from(modes))
    world = 1 if mode == PLAIN else draw(st.sampled_from([1, 2, 3, 4, 8]))
    rank = draw(st.integers(0, world - 1))
    pair = draw(st.booleans())
    rows = 256 * draw(st.integers(1, 12)) if pair else draw(st.integers(1, 1500))
    Ns = _widths(draw, pair)
    if mode == RS:
        Ns = Ns[:1]
    last_dim = draw(st.booleans()) if mode != PLAIN else False
    return mode, world, rank, rows, Ns, int(last_dim), int(pair)


def _units(mode, world, rank, rows, Ns, last_dim, pair):
    """Schedule as a list of scheduling units; a unit is a list of tiles (two for a CTA pair)."""
    if not pair:
        return [[tuple(r)] for r in schedule(mode, world, rank, rows, Ns, last_dim)]
    a = schedule(mode, world, rank, rows, Ns, last_dim, 1, 0)
    b = schedule(mode, world, rank, rows, Ns, last_dim, 1, 1)
    return [[tuple(x), tuple(y)] for x, y in zip(a, b)]


@settings(max_examples=150, deadline=None)
@given(_shapes())
def test_every_tile_is_scheduled_exactly_once(shape):
    mode, world, rank, rows, Ns, last_dim, pair = shape
    bn = 128 if max(Ns) <= 128 else 256
    units = _units(*shape)
    tiles = [t for u in units for t in u]
    chunks = range(world) if mode != PLAIN and not (mode == AG and last_dim) else range(1)
    want = expected_tiles(world, rows, Ns, bn, chunks)
    assert len(tiles) == len(want) and {t[:4] for t in tiles} == want
    mt = -(-rows // 128)
    per_chunk = len(want) // len(chunks)
    seen = set()
    for chunk, m, b, n0, tile_in_chunk, rows_valid in tiles:
        assert 0 <= tile_in_chunk < per_chunk                       # indexes flags and arena blocks of one chunk
        assert (chunk, tile_in_chunk) not in seen                   # ... without collisions
        seen.add((chunk, tile_in_chunk))
        assert rows_valid == (128 if m < mt - 1 or rows % 128 == 0 else rows % 128)
        assert n0 % bn == 0 and 0 <= n0 < Ns[b]


@settings(max_examples=60, deadline=None)
@given(_shapes(modes=(RS,)), st.sampled_from([0, 1, 2, 5, 14, 40]))
def test_reduce_scatter_waits_only_on_earlier_positions(shape, lag):
    """Progress argument of the reduce-scatter: a unit that owns its tile waits for the peers'
    partials of the same tile. On every peer that tile sits at an EARLIER position of the peer's
    list, and sends never wait on anything, so by induction over positions no set of co-resident
    CTAs can wait on each other in a cycle."""
    mode, world, rank, rows, Ns, last_dim, pair = shape
    if world == 1:
        return
    build_native()
    nat.lib().apk_debug_set_rs_lag(lag)       # launches size the lag from the grid; every value must keep the order safe
    try:
        per_rank = [_units(mode, world, r, rows, Ns, last_dim, pair) for r in range(world)]
    finally:
        nat.lib().apk_debug_set_rs_lag(0)
    want = expected_tiles(world, rows, Ns, 128 if max(Ns) <= 128 else 256, range(world))
    assert all({t[:4] for u in units for t in u} == want for units in per_rank)      # still an exact cover
    pos = [{t[:4]: i for i, u in enumerate(units) for t in u} for units in per_rank]
    ident = [{t[:4]: t[4] for u in units for t in u} for units in per_rank]
    for r in range(world):
        for i, unit in enumerate(per_rank[r]):
            for t in unit:
                if t[0] != r:
                    continue
                for s in range(world):
                    if s != r:
                        assert pos[s][t[:4]] < i, (r, s, t)
                        assert ident[s][t[:4]] == t[4]           # both sides name the tile's flag alike
    # all ranks walk lists of the same length with own / remote tiles at the same positions
    kinds = [[u[0][0] == r for u in per_rank[r]] for r in range(world)]
    assert all(k == kinds[0] for k in kinds)


@settings(max_examples=60, deadline=None)
@given(_shapes(modes=(AG,)))
def test_all_gather_starts_on_local_rows(shape):
    mode, world, rank, rows, Ns, last_dim, pair = shape
    units = _units(*shape)
    if last_dim:
        assert all(t[0] == 0 for u in units for t in u)             # one pass; K slices switch sources inside a tile
        return
    own = [i for i, u in enumerate(units) if u[0][0] == rank]
    assert own == list(range(len(own)))                             # nothing to wait for at the start
    assert len(own) * world == len(units)
