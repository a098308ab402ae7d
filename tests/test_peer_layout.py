"""Ownership and staging layout of the fused row-parallel sum (host arithmetic, no GPU):
a numpy model of "every rank stores its partial rows into the owner's slab, every owner
adds its slabs and hands the rows to everyone" must reproduce the plain sum."""

import numpy as np
import pytest

from dpk_b200 import peer


@pytest.mark.parametrize("M,world", [(1, 1), (127, 2), (128, 2), (129, 2), (2100, 4), (16384, 8),
                                     (1000, 8), (5, 8)])
def test_rows_per_owner_covers_all_rows_in_whole_windows(M, world):
    R = peer.rows_per_owner(M, world)
    assert R % peer.WINDOW == 0 and R * world >= M
    # a 128-token window never straddles two owners
    for w0 in range(0, M, peer.WINDOW):
        last = min(w0 + peer.WINDOW, M) - 1
        assert peer.owner_of_row(w0, M, world) == peer.owner_of_row(last, M, world)
    assert peer.owner_of_row(M - 1, M, world) < world
    # no smaller window multiple would do
    assert (R - peer.WINDOW) * world < M


def test_world_limits():
    with pytest.raises(ValueError):
        peer.rows_per_owner(10, 0)
    with pytest.raises(ValueError):
        peer.rows_per_owner(10, peer.MAX_WORLD + 1)


@pytest.mark.parametrize("M,world,ld", [(300, 2, 8), (700, 4, 16), (1030, 8, 8)])
def test_scatter_then_reduce_gather_is_the_sum(M, world, ld):
    rng = np.random.default_rng(M)
    partial = rng.standard_normal((world, M, ld)).astype(np.float32)
    R = peer.rows_per_owner(M, world)
    stage = np.full((world, world * R * ld), np.nan, dtype=np.float32)     # [owner][slabs]
    for src in range(world):
        for row in range(M):
            o = peer.owner_of_row(row, M, world)
            off = peer.slab_offset(row, M, world, src, ld)
            stage[o, off:off + ld] = partial[src, row]
    out = np.full((world, M, ld), np.nan, dtype=np.float32)
    for o in range(world):
        slabs = stage[o].reshape(world, R, ld)
        rows = max(0, min(R, M - o * R))
        total = slabs[:, :rows].sum(axis=0)
        for dst in range(world):
            out[dst, o * R:o * R + rows] = total
    want = partial.sum(axis=0)
    for dst in range(world):
        np.testing.assert_allclose(out[dst], want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("M,world", [(1024, 2), (2100, 4), (4500, 8), (16384, 8), (8192, 8), (513, 2), (100000, 8)])
def test_two_halves_cover_the_rows_and_fit_the_staging_buffer(M, world):
    width = 8
    r0, n0, s0 = peer.half_split(M, world, width, 0)
    r1, n1, s1 = peer.half_split(M, world, width, 1)
    assert (r0, s0) == (0, 0) and r1 == n0 and n0 + n1 == M
    assert n0 % peer.WINDOW == 0 or n1 == 0                 # the cut is on a window boundary
    # the second half's slabs start right after the first half's and both fit what connect() sizes
    assert s1 == world * peer.rows_per_owner(n0, world) * width
    end = s1 + world * peer.rows_per_owner(max(n1, 1), world) * width
    assert end <= world * peer.staging_rows(M, world) * width
    assert peer.half_split(M, world, width, None) == (0, M, 0)
