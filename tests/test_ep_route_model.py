"""The one-launch route sort of the expert-parallel block (csrc/ep.cu: ep_route_kernel) restated step by
step (passes of 1024 routes, 32 warps, match masks inside a warp, a scan over the warps, running totals
across passes) and compared with a stable counting sort (counting_sort, src/ops/moe.rs:463-508) on random
routing tables of awkward sizes.  This checks the algorithm, not the CUDA code; the kernel itself meets
the oracle in tests/test_gpu_ep.py (one and two passes)."""
import numpy as np
import pytest


def route_kernel_model(all_inds, base, e_local, block=1024):
    routes = len(all_inds)
    local = lambda i: (int(all_inds[i]) - base) if (i < routes and 0 <= int(all_inds[i]) - base < e_local) else -1
    counts = np.zeros(e_local + 1, np.int64)
    for i in range(routes):
        if local(i) >= 0:
            counts[local(i)] += 1
    seg = np.zeros(e_local + 1, np.int64)          # exclusive scan, 32 experts per step with a carry
    carry = 0
    for e0 in range(0, e_local + 1, 32):
        c = np.array([counts[e] if e < e_local else 0 for e in range(e0, e0 + 32)])
        incl = np.cumsum(c)
        for lane in range(32):
            if e0 + lane <= e_local:
                seg[e0 + lane] = carry + incl[lane] - c[lane]
        carry += incl[31]
    perm = np.full(int(seg[e_local]), -1, np.int64)
    done = np.zeros(e_local, np.int64)
    for i0 in range(0, routes, block):
        cnt = np.zeros((block // 32, e_local), np.int64)
        e_of = [local(i0 + t) for t in range(block)]
        rank_in_warp = [0] * block
        for w in range(block // 32):
            lanes = e_of[32 * w:32 * w + 32]
            for lane, e in enumerate(lanes):
                same = [l for l in range(32) if lanes[l] == e]          # __match_any_sync
                rank_in_warp[32 * w + lane] = sum(1 for l in same if l < lane)
                if e >= 0 and rank_in_warp[32 * w + lane] == 0:
                    cnt[w][e] = len(same)
        off = np.zeros_like(cnt)
        for x in range(e_local):                                          # scan over the warps
            acc = done[x]
            for w in range(block // 32):
                off[w][x] = acc
                acc += cnt[w][x]
            done[x] = acc
        for t in range(block):
            e = e_of[t]
            if e >= 0:
                perm[seg[e] + off[t // 32][e] + rank_in_warp[t]] = i0 + t
    return seg, perm


@pytest.mark.parametrize("routes,E,world,rank", [(80, 16, 2, 1), (1024, 256, 1, 0), (1600, 256, 1, 0), (2049, 64, 4, 2),
                                                 (33, 8, 8, 7), (1, 256, 1, 0), (3000, 32, 1, 0)])
def test_route_sort_is_a_stable_counting_sort(routes, E, world, rank):
    rng = np.random.default_rng(routes * 7 + E)
    inds = rng.integers(0, E, routes)
    el = E // world
    seg, perm = route_kernel_model(inds, rank * el, el)
    mine = [i for i in range(routes) if rank * el <= inds[i] < (rank + 1) * el]
    want = sorted(mine, key=lambda i: (inds[i], i))                       # stable by expert, then by route
    assert list(perm) == want
    for e in range(el):
        assert seg[e] == sum(1 for i in mine if inds[i] - rank * el < e)
    assert seg[el] == len(mine)
