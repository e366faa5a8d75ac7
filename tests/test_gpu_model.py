"""The CUDA model and generation loops against the CPU oracle (tiny model), and
size-independent properties at the real dimensions."""
import numpy as np
import pytest

import helpers as hp
import orn_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny(pkg, ctx):
    cfg = hp.tiny_config(pkg.Config)
    W = hp.tiny_model_weights(cfg, seed=5)
    om = orc.Model(cfg, W)
    gm = hp.upload_model(pkg, ctx, cfg, W)
    yield cfg, W, om, gm
    gm.free()
    om.free()


def test_forward_matches_oracle(pkg, ctx, tiny):
    cfg, W, om, gm = tiny
    ids = np.array([3, 77, 1500, 9, 12, 800, 41], np.uint32)
    oc = om.new_cache()
    gc = gm.make_cache()
    for a, b in [(0, 1), (1, 3), (3, 7)]:
        ref = om.forward(oc, ids[a:b])
        got = gm.forward(gc, ids[a:b]).numpy()
        assert np.array_equal(got, ref), (a, b)
    assert gc.offset == 7
    # logits and greedy tokens of the last rows
    rt, rl = om.head_greedy(ref, 4, want_logits=True)
    gt, gl = gm.head_greedy(ctx.upload(ref), 4, want_logits=True)
    assert np.array_equal(gl.numpy(), rl) and gt.tolist() == rt.tolist()
    om.free_cache(oc)
    gc.free()


def test_capture_and_rewind(pkg, ctx, tiny):
    """forward_capture + rewind(keep) leaves the caches as if only `keep`
    tokens had been stepped (tests/mtp.rs:177-234)."""
    cfg, W, om, gm = tiny
    ids = np.array([10, 20, 30, 40, 50], np.uint32)
    for keep in (1, 2):
        a, b = gm.make_cache(), gm.make_cache()
        gm.forward(a, ids[:2])
        gm.forward(b, ids[:2])
        gm.forward(a, ids[2:4], capture=True)
        a.rewind(keep)
        for t in range(keep):
            gm.forward(b, ids[2 + t:3 + t])
        assert a.offset == b.offset == 2 + keep
        ya = gm.forward(a, ids[4:5]).numpy()
        yb = gm.forward(b, ids[4:5]).numpy()
        assert np.array_equal(ya, yb)
        a.free()
        b.free()


def test_generate_matches_oracle(pkg, ctx, tiny):
    cfg, W, om, gm = tiny
    prompt = np.array([5, 900, 33, 1201, 8, 64, 700], np.uint32)
    ref = om.generate(prompt, 24)
    c = gm.make_cache()
    got = pkg.generate_step(gm, c, prompt, 24)
    assert got == ref
    assert c.offset == len(prompt) + 24
    # on_token returning False stops, the stopping token included
    seen = []
    c.reset()
    out = pkg.generate_step(gm, c, prompt, 24, on_token=lambda t: (seen.append(t) or len(seen) < 5))
    assert out == ref[:5] and c.offset == len(prompt) + 5
    c.free()


@pytest.mark.parametrize("policy", [0, 1])
@pytest.mark.parametrize("p", [0.0, 0.5, 0.9])
def test_mtp_matches_oracle_and_autoregressive(pkg, ctx, tiny, policy, p):
    """BASELINE config 4 on the tiny model: emitted ids byte-identical to the
    non-speculative run, accepted counts equal to the oracle's."""
    cfg, W, om, gm = tiny
    prompt = np.array([5, 900, 33, 1201, 8, 64, 700], np.uint32)
    ar = om.generate(prompt, 30)
    force = (ar, p, 42) if p > 0 else None
    ref, rst = om.generate_mtp(prompt, 1, 30, policy=policy, force=force)
    c = gm.make_cache()
    got, gst = pkg.generate_step_mtp(gm, c, prompt, 1, 30, policy=policy, force=force)
    assert got == ar == ref
    assert (gst.cycles, gst.drafted, gst.accepted) == (rst.cycles, rst.drafted, rst.accepted)
    assert list(gst.accepted_by_depth) == list(rst.accepted_by_depth)
    assert c.offset == len(prompt) + 30
    c.free()


def test_mtp_depth2_and_frspec(pkg, ctx, tiny):
    cfg, W, om, gm = tiny
    prompt = np.array([1, 2, 3, 4], np.uint32)
    ar = om.generate(prompt, 16)
    rng = np.random.default_rng(0)
    ids = np.sort(rng.choice(cfg.vocab, 512, replace=False)).astype(np.uint32)
    om.set_frspec(hp.gather_rows_weights(W["lm_head"], ids), ids)
    gm.set_frspec(ids)
    c = gm.make_cache()
    for depth, fr in [(2, False), (1, True), (3, True)]:
        c.reset()
        ref, rst = om.generate_mtp(prompt, depth, 16, policy=1, frspec=fr, force=(ar, 0.7, 9))
        got, gst = pkg.generate_step_mtp(gm, c, prompt, depth, 16, policy=1, frspec=fr, force=(ar, 0.7, 9))
        assert got == ar == ref
        assert (gst.cycles, gst.drafted, gst.accepted) == (rst.cycles, rst.drafted, rst.accepted)
    c.free()
    # bad id lists are refused (src/frspec.rs:78-100)
    with pytest.raises(pkg.OrnError):
        gm.set_frspec(np.array([1, 1], np.uint32))
    with pytest.raises(pkg.OrnError):
        gm.set_frspec(np.array([cfg.vocab], np.uint32))


def test_load_from_safetensors_artifact(pkg, ctx, tiny, tmp_path):
    """orn_model_load (config.json, sharded safetensors + index, MTP sidecar with numbered experts) and
    orn_frspec_load give the same model as uploading the tensors one by one."""
    cfg, W, om, gm = tiny
    rng = np.random.default_rng(3)
    ids = np.sort(rng.choice(cfg.vocab, 256, replace=False)).astype(np.uint32)
    d = hp.write_artifact(str(tmp_path / "artifact"), cfg, W, frspec_ids=ids)
    lm = pkg.TextModel.load(ctx, d, max_ctx=cfg.max_ctx)
    for f in ("hidden", "n_layers", "n_heads", "n_kv_heads", "head_dim", "rope_dims", "gdn_k_heads", "gdn_v_heads",
              "n_experts", "top_k", "expert_inter", "shared_inter", "vocab", "full_attn_interval", "norm_topk_prob"):
        assert getattr(lm.cfg, f) == getattr(cfg, f), f
    prompt = np.array([11, 4, 1300, 77, 5], np.uint32)
    ref = om.generate(prompt, 12)
    c = lm.make_cache()
    assert pkg.generate_step(lm, c, prompt, 12) == ref
    c.reset()
    got, st = pkg.generate_step_mtp(lm, c, prompt, 2, 12)
    rref, rst = om.generate_mtp(prompt, 2, 12)
    assert got == ref == rref and (st.cycles, st.accepted) == (rst.cycles, rst.accepted)
    # FR-Spec ids file: the pruned head drafts the same as the oracle's
    om.set_frspec(hp.gather_rows_weights(W["lm_head"], ids), ids)
    lm.load_frspec(d + "/ids.bin")
    c.reset()
    got, st = pkg.generate_step_mtp(lm, c, prompt, 1, 12, frspec=True)
    rref, rst = om.generate_mtp(prompt, 1, 12, frspec=True)
    assert got == ref == rref and (st.cycles, st.accepted) == (rst.cycles, rst.accepted)
    c.free()
    lm.free()
    # a missing shard is an error code with a message, not a crash
    import os
    os.remove(d + "/model-00002-of-00002.safetensors")
    with pytest.raises(pkg.OrnError):
        pkg.TextModel.load(ctx, d, max_ctx=cfg.max_ctx)


def test_published_mix_loads_through_the_quantization_block(pkg, ctx, tmp_path):
    """The module formats of the reference's q6k-full artifact (tools/forge_q4k.py:131-152): Q4_K
    gated-delta projections, lm_head and routed experts (down included), Q6_K attention and
    routers, affine 4-bit group-32 shared experts, 8-bit affine embedding and shared-expert gates.
    config.json's `quantization` block names each module's mode (src/weights.rs:49-79,179-184): the
    default is affine 4-bit group 32, every other module is an override.  The MoE blocks fall out
    of the fused kernels' formats and run one kernel per op; tokens equal the oracle's."""
    cfg = hp.tiny_config(pkg.Config)
    W = hp.tiny_model_weights(cfg, seed=8, mix="published")
    kinds = {w.kind for w in W.values() if isinstance(w, orc.Weights)}
    assert kinds == {orc.Q4K, orc.Q6K, orc.A8, orc.A4, orc.BF16}
    om = orc.Model(cfg, W)
    d = hp.write_artifact(str(tmp_path / "published"), cfg, W, quant_block=True)
    lm = pkg.TextModel.load(ctx, d, max_ctx=cfg.max_ctx)
    assert lm.get_linear("layers.0.mlp.shared_expert.up_proj").kind == pkg.A4
    assert lm.get_linear("layers.0.mlp.gate").kind == pkg.Q6K
    assert lm.get_linear("layers.0.mlp.switch_mlp.down_proj").kind == pkg.Q4K
    prompt = np.array([11, 4, 1300, 77, 5, 900], np.uint32)
    ref = om.generate(prompt, 14)
    c = lm.make_cache()
    assert pkg.generate_step(lm, c, prompt, 14) == ref
    c.reset()
    got, st = pkg.generate_step_mtp(lm, c, prompt, 1, 14, force=(ref, 0.5, 2))
    rref, rst = om.generate_mtp(prompt, 1, 14, force=(ref, 0.5, 2))
    assert got == ref == rref and (st.cycles, st.accepted) == (rst.cycles, rst.accepted)
    # a long prompt takes the wide path: every format through the tensor-core product
    c.reset()
    long_ids = np.random.default_rng(1).integers(0, cfg.vocab, 70).astype(np.uint32)
    h = lm.prefill(c, long_ids, want_hidden=True).numpy()
    assert c.offset == 70 and np.isfinite(hp.bf16_to_f32(h)).all()
    c.free()
    lm.free()
    om.free()
    # a module whose tensors disagree with the block is refused at load
    import json
    cj = json.load(open(d + "/config.json"))
    cj["quantization"]["language_model.model.layers.0.mlp.gate"] = {"mode": "affine", "group_size": 64, "bits": 8}
    json.dump(cj, open(d + "/config.json", "w"))
    with pytest.raises(pkg.OrnError, match="affine module"):
        pkg.TextModel.load(ctx, d, max_ctx=cfg.max_ctx)
    cj["quantization"]["language_model.model.layers.0.mlp.gate"] = {"mode": "nvfp4", "group_size": 16, "bits": 4}
    json.dump(cj, open(d + "/config.json", "w"))
    with pytest.raises(pkg.OrnError, match="not on this path"):
        pkg.TextModel.load(ctx, d, max_ctx=cfg.max_ctx)


def test_truncated_tensor_is_refused(pkg, ctx, tmp_path):
    """A safetensors header whose shape asks for more bytes than data_offsets hold is an error at
    load, not a read past the mapping."""
    import json
    cfg = hp.tiny_config(pkg.Config)
    W = hp.tiny_model_weights(cfg, seed=5)
    d = hp.write_artifact(str(tmp_path / "trunc"), cfg, W)
    path = d + "/model-00001-of-00002.safetensors"
    raw = open(path, "rb").read()
    n = int.from_bytes(raw[:8], "little")
    hdr = json.loads(raw[8:8 + n])
    name = next(k for k, v in hdr.items() if v["dtype"] == "BF16" and len(v["shape"]) == 1)
    hdr[name]["shape"] = [hdr[name]["shape"][0] * 4]   # claims four times the bytes it has
    hj = json.dumps(hdr).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    open(path, "wb").write(len(hj).to_bytes(8, "little") + hj + raw[8 + n:])
    with pytest.raises(pkg.OrnError, match="do not match"):
        pkg.TextModel.load(ctx, d, max_ctx=cfg.max_ctx)


def test_full_size_layers_mtp_equals_autoregressive(pkg, ctx):
    """Real layer dimensions (hidden 2048, 256 experts top-8, 16/2 heads, vocab
    248320) at 4 layers, random-init on the GPU: speculative output is
    byte-identical to non-speculative output on the engine itself."""
    cfg = pkg.qwen35_config(max_ctx=160, n_layers=4)
    m = pkg.TextModel(ctx, cfg)
    m.init_random(7)
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, cfg.vocab, 9).astype(np.uint32)
    c = m.make_cache()
    ar = pkg.generate_step(m, c, prompt, 40)
    assert len(set(ar)) > 3  # not a degenerate stream
    for p in (0.0, 0.9):
        c.reset()
        got, st = pkg.generate_step_mtp(m, c, prompt, 1, 40, force=(ar, p, 5) if p else None)
        assert got == ar
        if p:
            assert st.accepted >= st.drafted // 2
    # FR-Spec with a seeded sorted unique subset of 65536 ids
    ids = np.sort(rng.choice(cfg.vocab, 65536, replace=False)).astype(np.uint32)
    m.set_frspec(ids)
    c.reset()
    got, st = pkg.generate_step_mtp(m, c, prompt, 1, 40, frspec=True, force=(ar, 0.5, 6))
    assert got == ar
    c.free()
    m.free()


def test_decode_past_the_split_attention_threshold_equals_the_oracle(pkg, ctx):
    """From 512 cached keys on the fused attention spreads the key groups of a head over four CTAs and
    merges their partials in the last one: same arithmetic, same bits.  A 503-token prompt through
    the row-invariant windows, then 24 generated tokens (autoregressive and MTP depth 1 and 2, so
    that windows of 1, 2 and 3 rows cross the threshold): ids, acceptance counts and hidden rows against
    the oracle.  The MTP head's own cache stays short here; its long form is the same kernel."""
    cfg = hp.tiny_config(pkg.Config, max_ctx=700)
    W = hp.tiny_model_weights(cfg, seed=15)
    om = orc.Model(cfg, W)
    gm = hp.upload_model(pkg, ctx, cfg, W)
    rng = np.random.default_rng(77)
    prompt = rng.integers(0, cfg.vocab, 503).astype(np.uint32)
    ar = om.generate(prompt, 24)
    c = gm.make_cache()
    assert pkg.generate_step(gm, c, prompt, 24, prefill_step=8) == ar
    for depth in (1, 2):
        ref, rst = om.generate_mtp(prompt, depth, 24, policy=1, force=(ar, 0.6, 5))
        c.reset()
        got, gst = pkg.generate_step_mtp(gm, c, prompt, depth, 24, prefill_step=8, force=(ar, 0.6, 5))
        assert got == ar == ref
        assert (gst.cycles, gst.drafted, gst.accepted) == (rst.cycles, rst.drafted, rst.accepted)
    # hidden rows of windows on both sides of the threshold
    oc = om.new_cache()
    c.reset()
    seq = np.concatenate([prompt, np.array(ar, np.uint32)])
    for a in range(0, 508, 4):
        ids = seq[a:a + 4]
        want = om.forward(oc, ids)
        got = gm.forward(c, ids).numpy()
        if a >= 488:
            assert np.array_equal(got, want), a
    for T in (3, 2, 1, 4, 2, 4, 4, 4, 4, 4, 4, 4, 4, 3):   # 508 .. 555: short form, the crossing window, long form
                                                           # with whole blocks of keys and every tail length
        ids = rng.integers(0, cfg.vocab, T).astype(np.uint32)
        assert np.array_equal(gm.forward(c, ids).numpy(), om.forward(oc, ids)), (T, c.offset)
    om.free_cache(oc)
    c.free()
    gm.free()
    om.free()
