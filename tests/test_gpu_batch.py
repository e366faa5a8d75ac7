"""Batched decode (csrc/batch.cu) against the single-sequence engine.

Exact mode: every sequence of a batch, stepping windows of 1 or 2 rows with its own acceptance
pattern, must reproduce the single-sequence engine's hidden rows and greedy targets bit for bit
(same kernels with a sequence index in their grids).  Tensor-core mode (16 rows and more): same
caches and inputs as an exact run, rows agree to the rounding of the products; the split-KV
attention is additionally checked against the exact kernel with every other product exact."""
import numpy as np
import pytest

import helpers as hp

pytestmark = pytest.mark.gpu


def bf(a):
    return hp.bf16_to_f32(a)


def run_single(pkg, gm, windows, keeps, b):
    """sequence b alone through forward_capture / rewind; returns the hidden rows and targets per window"""
    c = gm.make_cache()
    out = []
    for w, k in zip(windows, keeps):
        ids = np.ascontiguousarray(w[b], np.uint32)
        h = gm.forward(c, ids, capture=True)
        toks = gm.head_greedy(h, len(ids))
        out.append((h.numpy().copy(), toks.copy()))
        c.rewind(int(k[b]))
    c.free()
    return out


def test_batched_exact_equals_the_single_sequence_engine(pkg, ctx):
    cfg = hp.tiny_config(pkg.Config)
    W = hp.tiny_model_weights(cfg, seed=11)
    gm = hp.upload_model(pkg, ctx, cfg, W)
    rng = np.random.default_rng(3)
    B = 3
    shapes = [2, 2, 1, 2, 2, 1, 2]
    windows = [rng.integers(0, cfg.vocab, (B, t)).astype(np.uint32) for t in shapes]
    keeps = [np.array([rng.integers(1, t + 1) for _ in range(B)], np.int32) for t in shapes]
    bt = pkg.Batch(gm, B, t_max=2, cap=64, exact=True)
    got = []
    for w, k in zip(windows, keeps):
        tg, hid = bt.forward(w, want_hidden=True)
        got.append((hid.numpy().reshape(B, w.shape[1], cfg.hidden).copy(), tg.copy()))
        bt.commit(k)
    assert list(bt.positions()) == [int(sum(k[b] for k in keeps)) for b in range(B)]
    for b in range(B):
        want = run_single(pkg, gm, windows, keeps, b)
        for i, ((wh, wt), (gh, gt)) in enumerate(zip(want, got)):
            assert np.array_equal(wh.reshape(-1, cfg.hidden), gh[b]), (b, i)
            assert np.array_equal(wt, gt[b]), (b, i)
    # reset returns every sequence to an empty cache
    bt.reset()
    tg, hid = bt.forward(windows[0], want_hidden=True)
    assert np.array_equal(hid.numpy().reshape(B, 2, cfg.hidden), got[0][0])
    bt.free()
    gm.free()


def test_batched_exact_full_width_layers(pkg, ctx):
    cfg = pkg.qwen35_config(max_ctx=64, n_layers=4)
    gm = pkg.TextModel(ctx, cfg)
    gm.init_random(21)
    rng = np.random.default_rng(5)
    B = 2
    windows = [rng.integers(0, cfg.vocab, (B, 2)).astype(np.uint32) for _ in range(3)]
    keeps = [np.array([2, 1], np.int32), np.array([1, 2], np.int32), np.array([2, 2], np.int32)]
    bt = pkg.Batch(gm, B, t_max=2, cap=32, exact=True)
    got = []
    for w, k in zip(windows, keeps):
        tg, hid = bt.forward(w, want_hidden=True)
        got.append((hid.numpy().reshape(B, 2, cfg.hidden).copy(), tg.copy()))
        bt.commit(k)
    for b in range(B):
        want = run_single(pkg, gm, windows, keeps, b)
        for i, ((wh, wt), (gh, gt)) in enumerate(zip(want, got)):
            assert np.array_equal(wh.reshape(-1, cfg.hidden), gh[b]), (b, i)
            assert np.array_equal(wt, gt[b]), (b, i)
    bt.free()
    gm.free()


def row_stats(want, got):
    w, g = bf(want).astype(np.float64), bf(got).astype(np.float64)
    cos = (w * g).sum(-1) / np.sqrt((w * w).sum(-1) * (g * g).sum(-1) + 1e-30)
    err = np.abs(w - g).max(-1) / (np.abs(w).max(-1) + 1e-30)
    return cos, err


@pytest.mark.parametrize("ctx_len", [0, 300])
def test_batched_tensor_core_mode_agrees_with_exact_mode(pkg, ctx, ctx_len):
    """16 rows: projections, experts and lm_head on the tensor cores, attention split over the
    caches.  A routing flip is a discrete change, not an error, so agreement is statistical and per
    row: cosine and max error relative to the row's max."""
    cfg = hp.tiny_config(pkg.Config)
    W = hp.tiny_model_weights(cfg, seed=12)
    gm = hp.upload_model(pkg, ctx, cfg, W)
    B = 8
    ids = np.random.default_rng(9).integers(0, cfg.vocab, (B, 2)).astype(np.uint32)
    outs = {}
    for exact in (True, False):
        bt = pkg.Batch(gm, B, t_max=2, cap=640, exact=exact)
        if ctx_len:
            bt.fill_random(ctx_len, seed=7)
        tg, hid = bt.forward(ids, want_hidden=True)
        bt.commit(np.full(B, 2, np.int32))
        tg2, hid2 = bt.forward(ids[:, ::-1].copy(), want_hidden=True)
        outs[exact] = (hid.numpy().copy(), tg.copy(), hid2.numpy().copy(), tg2.copy())
        assert list(bt.positions()) == [ctx_len + 2] * B
        bt.free()
    for a, b, tol in ((0, 0, 0.03), (2, 2, 0.08)):     # the second window also inherits the first one's state
        cos, err = row_stats(outs[True][a], outs[False][b])
        assert np.median(cos) > 0.998, (ctx_len, a, np.sort(cos)[:4])
        assert np.median(err) < tol, (ctx_len, a, np.sort(err)[-4:])
        assert np.mean(cos > 0.995) >= 0.6, (ctx_len, a, np.sort(cos)[:4])   # a flipped route moves its whole sequence
    gm.free()


@pytest.mark.parametrize("ctx_len", [3, 300, 517])
def test_split_kv_attention_alone(pkg, ctx, ctx_len):
    """Every product exact, only the attention differs: one pass per (KV head, 256-key chunk)
    with an online softmax and a merge, against the kernel that walks the cache per query.  The two
    sum in a different order in f32, so hidden rows differ by a bf16 rounding here and there."""
    cfg = hp.tiny_config(pkg.Config)
    W = hp.tiny_model_weights(cfg, seed=13)
    gm = hp.upload_model(pkg, ctx, cfg, W)
    B = 5
    ids = np.random.default_rng(2).integers(0, cfg.vocab, (B, 2)).astype(np.uint32)
    outs = {}
    for split in (False, True):
        bt = pkg.Batch(gm, B, t_max=2, cap=640, exact=True, split_attn=split)
        bt.fill_random(ctx_len, seed=3)
        _, hid = bt.forward(ids, want_hidden=True)
        bt.commit(np.array([1, 2, 1, 2, 2], np.int32))     # ragged positions for the second window
        _, hid2 = bt.forward(ids, want_hidden=True)
        outs[split] = (hid.numpy().copy(), hid2.numpy().copy())
        bt.free()
    for i in range(2):
        cos, err = row_stats(outs[False][i], outs[True][i])
        assert np.median(err) < 0.01 and np.median(cos) > 0.9999, (i, err, cos)
        assert np.mean(cos > 0.9999) >= 0.8, (i, cos)
    gm.free()


def splitmix64(x):
    x = (x + 0x9e3779b97f4a7c15) & 0xFFFFFFFFFFFFFFFF
    x = ((x ^ (x >> 30)) * 0xbf58476d1ce4e5b9) & 0xFFFFFFFFFFFFFFFF
    x = ((x ^ (x >> 27)) * 0x94d049bb133111eb) & 0xFFFFFFFFFFFFFFFF
    return x ^ (x >> 31)


def forced(stream, p, seed, cycle, emitted):
    """the harness's forced draft for generated position emitted + 1 in this cycle, or None (orn_generate_step_mtp)"""
    if emitted + 1 >= len(stream):
        return None
    uni = (splitmix64(seed + cycle * 8) >> 40) / 16777216.0
    return int(stream[emitted + 1]) if uni < p else None


def test_batched_mtp_cycles_equal_the_single_sequence_engine(pkg, ctx):
    """MTP depth-1 decode of three sequences in lockstep (draft, verify window [primary, draft],
    per-sequence acceptance, Committed re-encode) against the single-sequence engine: the drafts and
    targets of every cycle against an op-level cycle of the same calls (orn_mtp_forward,
    orn_forward_capture, orn_cache_rewind), and the emitted tokens against orn_generate_step_mtp
    (itself compared with the oracle elsewhere).  Forced drafts (p = 0.6) make both acceptance
    outcomes occur; unforced cycles use the head's own draft."""
    cfg = hp.tiny_config(pkg.Config)
    W = hp.tiny_model_weights(cfg, seed=21)
    gm = hp.upload_model(pkg, ctx, cfg, W)
    rng = np.random.default_rng(17)
    B, NP, CYC, P = 3, 7, 9, 0.6
    prompts = rng.integers(0, cfg.vocab, (B, NP)).astype(np.uint32)
    seeds = [5, 6, 7]
    # the single-sequence engine: the autoregressive stream (the forced drafts come from it) and the MTP loop's output
    cache = gm.make_cache()
    ar, mtp = [], []
    for b in range(B):
        cache.reset()
        ar.append(pkg.generate_step(gm, cache, prompts[b], 30))
        cache.reset()
        toks, _ = pkg.generate_step_mtp(gm, cache, prompts[b], 1, 30, force=(ar[b], P, seeds[b]))
        assert toks == ar[b]
        mtp.append(toks)
    # the same cycles at op level on the single-sequence engine: drafts, targets, acceptance per cycle
    single = []
    for b in range(B):
        cache.reset()
        gm.forward(cache, prompts[b][:4])
        gm.forward(cache, prompts[b][4:NP - 1])
        h = gm.forward(cache, prompts[b][NP - 1:])
        primary = int(gm.head_greedy(h, 1)[0])
        hrow = ctx.upload(h.numpy()[0:1].copy())
        ctx.check(ctx._lib.orn_cache_set_mtp_offset(cache.h, 0), "mtp offset")
        emitted, log = 0, []
        for cyc in range(CYC):
            off = ctx._lib.orn_cache_mtp_offset(cache.h)
            draft = gm.mtp_forward(cache, hrow, [primary])
            f = forced(ar[b], P, seeds[b], cyc, emitted)
            used = draft if f is None else f
            vh = gm.forward(cache, np.array([primary, used], np.uint32), capture=True)
            tg = gm.head_greedy(vh, 2)
            k = 1 if int(tg[0]) == used else 0
            cache.rewind(k + 1)
            ctx.check(ctx._lib.orn_cache_set_mtp_offset(cache.h, off + 1), "mtp offset")
            if k:
                gm.mtp_forward(cache, vh, [used], kv_only=True)
            hrow = ctx.upload(vh.numpy()[k:k + 1].copy())
            log.append((draft, used, [int(t) for t in tg], k))
            emitted += k + 1
            primary = int(tg[k])
        single.append(log)
    cache.free()
    # the batched engine, exact arithmetic
    bt = pkg.Batch(gm, B, t_max=2, cap=96, exact=True)
    for a in range(0, NP - 1, 2):
        bt.forward(prompts[:, a:a + 2], want_targets=False)
        bt.commit(np.full(B, 2, np.int32))
    tg, _ = bt.forward(prompts[:, NP - 1:])
    bt.commit(np.ones(B, np.int32))
    primary = tg[:, 0].copy()
    emitted = [0] * B
    out = [[] for _ in range(B)]
    for cyc in range(CYC):
        drafts = bt.mtp_draft(primary)
        used = drafts.copy()
        for b in range(B):
            f = forced(ar[b], P, seeds[b], cyc, emitted[b])
            if f is not None:
                used[b] = f
        tg, _ = bt.forward(np.stack([primary, used], 1))
        k = (tg[:, 0] == used).astype(np.int32)
        bt.commit(k + 1)
        for b in range(B):
            want = single[b][cyc]
            assert (int(drafts[b]), int(used[b]), [int(t) for t in tg[b]], int(k[b])) == want, (b, cyc)
            out[b].append(int(primary[b]))
            if k[b]:
                out[b].append(int(used[b]))
            emitted[b] += int(k[b]) + 1
            primary[b] = tg[b, k[b]]
    ks = [x[3] for log in single for x in log]
    assert 0 < sum(ks) < len(ks)          # both acceptance outcomes occurred
    for b in range(B):
        assert out[b] == mtp[b][:len(out[b])], b
    bt.free()
    gm.free()
