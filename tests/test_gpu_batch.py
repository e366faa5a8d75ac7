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
