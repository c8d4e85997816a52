"""Tile enumeration and classification (csrc/geometry.h) through the C ABI's host-only probes, against the
oracle's materialised mask: every visible pair is covered by an enumerated tile, every tile called "full" is
fully visible, every tile called "skip" is fully hidden. No GPU needed."""

import ctypes as C

import numpy as np
import pytest

from fast_diffusion_attention import _lib
from oracle import diffusion_oracle as orc

CASES = [(n, bs) for n in (1, 2, 5, 37, 64, 100, 128, 129, 255, 256, 300, 517) for bs in (1, 2, 3, 7, 16, 64, 100, 128, 200, 256, 1024)]


def key_plan(lib, qh, qa, qb, n, bs, bn):
    cap = 4096
    hs, ts = (C.c_int32 * cap)(), (C.c_int32 * cap)()
    cnt = lib.fda_geom_key_plan(qh, qa, qb, n, bs, bn, hs, ts, cap)
    return [(hs[i], ts[i]) for i in range(cnt)]


def query_plan(lib, kh, k0, k1, n, bs, bm):
    cap = 4096
    hs, ts = (C.c_int32 * cap)(), (C.c_int32 * cap)()
    cnt = lib.fda_geom_query_plan(kh, k0, k1, n, bs, bm, hs, ts, cap)
    return [(hs[i], ts[i]) for i in range(cnt)]


def sub(vis, n, qh, qa, qb, kh, k0, k1):
    """visibility of query rows [qa,qb) of half qh vs keys [k0,k1) of half kh (keys past n are hidden)."""
    k1c = min(k1, n)
    block = np.zeros((qb - qa, k1 - k0), dtype=bool)
    if k1c > k0:
        block[:, : k1c - k0] = vis[(1 - 0) * 0 + (n if qh else 0) + qa:(n if qh else 0) + qb,
                                   (n if kh else 0) + k0:(n if kh else 0) + k1c]
    return block


@pytest.mark.parametrize("rows_per_item", [128, 256])
@pytest.mark.parametrize("n,bs", CASES)
def test_forward_enumeration(n, bs, rows_per_item):
    lib = _lib.load()
    vis = orc.visibility(n, bs).numpy()
    bn = 128
    for qh in (0, 1):
        for qa in range(0, n, rows_per_item):
            qb = min(qa + rows_per_item, n)
            steps = key_plan(lib, qh, qa, qb, n, bs, bn)
            assert len(set(steps)) == len(steps)
            covered = np.zeros((qb - qa, 2 * n), dtype=bool)
            for kh, kt in steps:
                k0 = kt * bn
                any_active = False
                for ta in range(qa, qb, 128):
                    tb = min(ta + 128, qb)
                    cls = lib.fda_geom_classify(qh, kh, ta, tb, k0, bn, n, bs, 128, 0)
                    blk = sub(vis, n, qh, ta, tb, kh, k0, k0 + bn)
                    if cls == 0:
                        assert not blk.any()
                    elif cls == 1:
                        assert blk.all()
                        any_active = True
                    else:
                        assert blk.any() and not blk.all()
                        any_active = True
                    if cls:
                        k1c = min(k0 + bn, n)
                        covered[ta - qa:tb - qa, (n if kh else 0) + k0:(n if kh else 0) + k1c] = True
                assert any_active, "a step nobody needs"
            want = vis[(n if qh else 0) + qa:(n if qh else 0) + qb]
            assert not (want & ~covered).any(), "visible pair not covered"


@pytest.mark.parametrize("n,bs", CASES)
def test_backward_enumeration(n, bs):
    lib = _lib.load()
    vis = orc.visibility(n, bs).numpy()
    bm = bn = 128
    for kh in (0, 1):
        for k0 in range(0, n, bn):
            k1 = min(k0 + bn, n)
            steps = query_plan(lib, kh, k0, k1, n, bs, bm)
            assert len(set(steps)) == len(steps)
            covered = np.zeros((2 * n, k1 - k0), dtype=bool)
            for qh, qt in steps:
                qa, qb = qt * bm, min(qt * bm + bm, n)
                assert qa < n
                cls = lib.fda_geom_classify(qh, kh, qa, qb, k0, bn, n, bs, bm, 1)
                blk = sub(vis, n, qh, qa, qb, kh, k0, k0 + bn)
                if cls == 0:
                    assert not blk.any()
                elif cls == 1:
                    assert blk.all()
                else:
                    assert blk.any() and not blk.all()
                if cls:
                    covered[(n if qh else 0) + qa:(n if qh else 0) + qb] = True
            want = vis[:, (n if kh else 0) + k0:(n if kh else 0) + k1]
            assert not (want & ~covered).any(), "visible pair not covered"


# ------------------------------------------------------------------------------------------------- item order
@pytest.mark.parametrize("per_group,n_groups,short8,ctas", [
    (32, 128, 4, 148),    # the benchmark's key tiles on one GPU: 27 items per block, groups one after the other
    (32, 16, 4, 148),     # an eighth of it: 3.5 items per block, rank for rank over all groups
    (16, 16, 2, 148),     # its forward items: fewer than two per block
    (1, 5, 1, 3), (7, 3, 8, 1), (5, 4, 0, 2), (64, 40, 1, 132),
])
def test_item_order_visits_every_item_once(per_group, n_groups, short8, ctas):
    """The order is a permutation of (group, rank); small launches go rank-major (every group's longest items
    first), large ones group-major with the short ranks of all groups at the end."""
    lib = _lib.load()
    g, r = C.c_int32(), C.c_int32()
    seen = []
    for idx in range(per_group * n_groups):
        assert lib.fda_geom_item_order(idx, per_group, n_groups, short8, ctas, C.byref(g), C.byref(r)) == 0
        assert 0 <= g.value < n_groups and 0 <= r.value < per_group
        seen.append((g.value, r.value))
    assert len(set(seen)) == per_group * n_groups
    total = per_group * n_groups
    if total <= 8 * ctas:
        assert seen == [(i % n_groups, i // n_groups) for i in range(total)]
    else:
        n_long = max(1, per_group - short8 * per_group // 8)
        head = seen[: n_long * n_groups]
        assert head == [(i // n_long, i % n_long) for i in range(n_long * n_groups)]
        assert all(rank >= n_long for _, rank in seen[n_long * n_groups:])
    # out of range
    assert lib.fda_geom_item_order(total, per_group, n_groups, short8, ctas, C.byref(g), C.byref(r)) == -1
    assert lib.fda_geom_item_order(0, 0, n_groups, short8, ctas, C.byref(g), C.byref(r)) == -1
