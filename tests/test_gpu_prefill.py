"""The prompt path: chunks of 64 rows or more run through the wide tensor-core products
(orn_gemm / the grouped expert product), shorter chunks through the row-invariant 4-row windows.
The reference exempts prefill from row invariance (src/generate.rs:99).  The chunk plumbing is
checked bit for bit with exact products in tests/test_gpu_fullwidth.py; here the tensor-core
products run, and the comparison with the row-invariant path (which other tests hold to the
oracle bit for bit) is statistical: every activation is re-rounded to bfloat16 between ops, a
random-init router has many near-ties, and one flipped expert changes a whole row."""
import numpy as np
import pytest

import helpers as hp
import orn_oracle as orc

pytestmark = pytest.mark.gpu


def row_errors(got, want):
    """per row: largest difference relative to the row's largest value, and the cosine"""
    g, w = hp.bf16_to_f32(got).astype(np.float64), hp.bf16_to_f32(want).astype(np.float64)
    rel = np.abs(g - w).max(1) / np.abs(w).max(1)
    cos = (g * w).sum(1) / np.sqrt((g * g).sum(1) * (w * w).sum(1))
    return rel, cos


@pytest.mark.parametrize("interval,what", [(4, "gated-delta layer"), (1, "attention layer")])
def test_one_layer_hidden_rows_within_rounding(pkg, ctx, interval, what):
    """One layer (mixer + MoE) on 70 rows: the typical row differs from the row-invariant path by
    a couple of bfloat16 steps of its largest value (<= 2e-2); rows whose routing flipped may
    differ more and are few."""
    cfg = hp.tiny_config(pkg.Config, max_ctx=160, n_layers=1, full_attn_interval=interval)
    W = hp.tiny_model_weights(cfg, seed=5)
    gm = hp.upload_model(pkg, ctx, cfg, W)
    ids = np.random.default_rng(4).integers(0, cfg.vocab, 70).astype(np.uint32)
    c = gm.make_cache()
    narrow = gm.prefill(c, ids, prefill_step=8, want_hidden=True).numpy()
    c.reset()
    wide = gm.prefill(c, ids, prefill_step=2048, want_hidden=True).numpy()
    assert c.offset == 70
    rel, cos = row_errors(wide, narrow)
    assert np.median(rel) <= 2e-2, np.median(rel)
    assert (rel > 5e-2).mean() <= 0.1
    assert np.median(cos) >= 0.9995
    c.free()
    gm.free()


def test_wide_prefill_and_generation_on_the_tiny_model(pkg, ctx):
    cfg = hp.tiny_config(pkg.Config, max_ctx=160)
    W = hp.tiny_model_weights(cfg, seed=5)
    om = orc.Model(cfg, W)
    gm = hp.upload_model(pkg, ctx, cfg, W)
    rng = np.random.default_rng(4)
    ids = rng.integers(0, cfg.vocab, 70).astype(np.uint32)
    oc = om.new_cache()
    ref = np.concatenate([om.forward(oc, ids[a:a + 4]) for a in range(0, 70, 4)])
    om.free_cache(oc)
    c = gm.make_cache()
    narrow = gm.prefill(c, ids, prefill_step=8, want_hidden=True).numpy()   # 8-row chunks: 4-row windows
    assert np.array_equal(narrow, ref)                                       # the row-invariant path is the oracle's
    for step in (2048, 64):   # one 70-row chunk; a 64-row chunk and a 6-row one (the last in windows)
        c.reset()
        wide = gm.prefill(c, ids, prefill_step=step, want_hidden=True).numpy()
        assert c.offset == 70
        rel, cos = row_errors(wide, ref)
        assert np.median(cos) >= 0.97, (step, np.median(cos))
    # the decode loop on the caches a wide prefill left: speculative output equals the engine's own
    # autoregressive output, whatever the prompt arithmetic was
    prompt = ids[:66]
    c.reset()
    ar = pkg.generate_step(gm, c, prompt, 24)                       # 65-row prompt chunk: wide
    c.reset()
    got, st = pkg.generate_step_mtp(gm, c, prompt, 1, 24, force=(ar, 0.5, 3))
    assert got == ar
    c.reset()
    assert pkg.generate_step(gm, c, prompt, 24, prefill_step=8) == om.generate(prompt, 24)   # windows: the oracle's stream
    c.free()
    gm.free()
    om.free()


def test_wide_prefill_at_full_width(pkg, ctx):
    """Real layer dimensions (4 layers): a 300-token prompt as one wide chunk against the same
    prompt through 4-row windows; the routed experts run grouped (2400 routes over 256 experts)."""
    cfg = pkg.qwen35_config(max_ctx=400, n_layers=4)
    m = pkg.TextModel(ctx, cfg)
    m.init_random(3)
    rng = np.random.default_rng(2)
    ids = rng.integers(0, cfg.vocab, 300).astype(np.uint32)
    c = m.make_cache()
    narrow = m.prefill(c, ids, prefill_step=4, want_hidden=True).numpy()
    c.reset()
    wide = m.prefill(c, ids, prefill_step=2048, want_hidden=True).numpy()
    rel, cos = row_errors(wide, narrow)
    assert np.median(cos) >= 0.97, np.median(cos)
    c.reset()
    ar = pkg.generate_step(m, c, ids, 12)
    c.reset()
    got, st = pkg.generate_step_mtp(m, c, ids, 1, 12, force=(ar, 0.5, 3))
    assert got == ar
    c.free()
    m.free()


def test_chunks_wider_than_2048_rows(pkg, ctx):
    """A 2600-token prompt as one chunk (prefill_step 4096), as 2048 + 552, and as 1000-row chunks: one
    layer of each kind on the tiny model.  Chunking changes which rows share a product launch and how
    the attention and the recurrence are cut, not what a row computes: the first chunk's rows of the
    2048 + 552 run equal the single chunk's bit for bit where the layer is causal-local (the
    gated-delta layer and everything per row), and all runs agree to rounding everywhere."""
    rng = np.random.default_rng(6)
    for interval in (4, 1):
        cfg = hp.tiny_config(pkg.Config, max_ctx=2700, n_layers=1, full_attn_interval=interval)
        gm = hp.upload_model(pkg, ctx, cfg, hp.tiny_model_weights(cfg, seed=8))
        ids = rng.integers(0, cfg.vocab, 2600).astype(np.uint32)
        c = gm.make_cache()
        outs = {}
        for step in (4096, 2048, 1000):
            c.reset()
            outs[step] = gm.prefill(c, ids, prefill_step=step, want_hidden=True).numpy()
            assert c.offset == 2600
        for step in (2048, 1000):
            rel, cos = row_errors(outs[step], outs[4096])
            assert np.median(cos) >= 0.999, (interval, step, np.median(cos))
            assert np.median(rel) <= 2e-2, (interval, step, np.median(rel))
        # the decode step continues from the caches of the one-chunk prompt
        c.reset()
        gm.prefill(c, ids, prefill_step=4096)
        h1 = gm.forward(c, ids[:2]).numpy()
        c.reset()
        gm.prefill(c, ids, prefill_step=1000)
        h2 = gm.forward(c, ids[:2]).numpy()
        rel, cos = row_errors(h1, h2)
        assert cos.min() >= 0.99, (interval, cos)
        c.free()
        gm.free()
