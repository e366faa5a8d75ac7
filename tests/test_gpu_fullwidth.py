"""The product path (persistent fused kernels, CUDA graphs) against the CPU oracle at the real
layer dimensions: hidden 2048, 256 experts top-8, 16 / 2 attention heads of 256, 16 / 32
gated-delta heads, vocab 248320, the benchmark's quantisation mix.  Four layers (three
gated-delta, one attention) stand for the forty: every kernel instantiation of the decode cycle
runs with the shapes it has in the full model."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers as hp
import orn_oracle as orc

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def full4(pkg, ctx):
    cfg = pkg.qwen35_config(max_ctx=96, n_layers=4)
    gm = pkg.TextModel(ctx, cfg)
    gm.init_random(20240611)
    gm.make_cache().free()  # resolves the weight table
    om = orc.export_gpu_model(gm)  # the same bytes on the CPU side
    yield cfg, om, gm
    gm.free()
    om.free()


def test_forward_windows_and_head_match_oracle(pkg, ctx, full4):
    """Hidden rows of 1-, 2- and 4-row windows (autoregressive step, verify window, prompt
    window), then logits and greedy tokens of the last four rows: bit for bit."""
    cfg, om, gm = full4
    rng = np.random.default_rng(3)
    ids = rng.integers(0, cfg.vocab, 9).astype(np.uint32)
    oc, gc = om.new_cache(), gm.make_cache()
    ref = None
    for a, b in [(0, 1), (1, 3), (3, 7), (7, 9)]:
        ref = om.forward(oc, ids[a:b])
        got = gm.forward(gc, ids[a:b]).numpy()
        assert np.array_equal(got, ref), (a, b)
    ref4 = om.forward(oc, ids[:4])
    got4 = gm.forward(gc, ids[:4]).numpy()
    assert np.array_equal(got4, ref4)
    rt, rl = om.head_greedy(ref4, 4, want_logits=True)
    gt, gl = gm.head_greedy(ctx.upload(ref4), 4, want_logits=True)
    assert np.array_equal(gl.numpy(), rl)
    assert gt.tolist() == rt.tolist()
    om.free_cache(oc)
    gc.free()


@pytest.mark.parametrize("p", [0.0, 0.5, 0.9])
def test_mtp_integer_contract_at_full_width(pkg, ctx, full4, p):
    """BASELINE config 4's contract at the real layer sizes: emitted ids, cycles, drafted,
    accepted and accepted-by-depth equal the oracle's under forced drafts with probability p,
    and the speculative stream equals the autoregressive one (src/mtp_generate.rs:236-316)."""
    cfg, om, gm = full4
    rng = np.random.default_rng(11)
    prompt = rng.integers(0, cfg.vocab, 6).astype(np.uint32)
    n = 14
    ar = om.generate(prompt, n)
    c = gm.make_cache()
    assert pkg.generate_step(gm, c, prompt, n) == ar
    force = (ar, p, 77) if p > 0 else None
    ref, rst = om.generate_mtp(prompt, 1, n, policy=1, force=force)
    c.reset()
    got, gst = pkg.generate_step_mtp(gm, c, prompt, 1, n, policy=1, force=force)
    assert got == ref == ar
    assert (gst.cycles, gst.drafted, gst.accepted) == (rst.cycles, rst.drafted, rst.accepted)
    assert list(gst.accepted_by_depth) == list(rst.accepted_by_depth)
    assert list(gst.reached_by_depth) == list(rst.reached_by_depth)
    if p == 0.9:
        assert gst.accepted >= gst.drafted // 2
    c.free()


@pytest.mark.parametrize("T", [1, 2])
def test_config2_moe_layer_256_experts_fused(pkg, ctx, T):
    """BASELINE config 2 at its full size through the kernels the decode step runs
    (router + shared gate/up launch, expert up with the routing in its prologue, expert down
    with the combine): 256 experts top-8, Q4_K gate/up [512,2048], Q6_K down [2048,512],
    affine-8 router, shared expert with its sigmoid gate; routing indices and outputs bit-exact."""
    rng = np.random.default_rng(200 + T)
    H, E, I, k = 2048, 256, 512, 8
    ws = {
        "gate": hp.make_weights(rng, orc.A8, 1, E, H),
        "sw_gate": hp.raw_q4k(rng, E, I, H), "sw_up": hp.raw_q4k(rng, E, I, H),
        "sw_down": hp.raw_q6k(rng, E, H, I),
        "sh_gate": hp.raw_q4k(rng, 1, I, H), "sh_up": hp.raw_q4k(rng, 1, I, H),
        "sh_down": hp.raw_q6k(rng, 1, H, I), "sh_egate": hp.make_weights(rng, orc.A8, 1, 1, H),
    }
    x = hp.f32_to_bf16(rng.standard_normal((T, H)).astype(np.float32))
    ref_out, ref_inds = orc.moe_block(ws, x, T, k, 1)
    L = {n: pkg.Linear.from_numpy(ctx, w.kind, w.w, w.s, w.b, E=w.E, O=w.O, K=w.K) for n, w in ws.items()}
    out, inds = ctx.empty((T, H), np.uint16), ctx.empty((T, k), np.uint32)
    order = ["gate", "sw_gate", "sw_up", "sw_down", "sh_gate", "sh_up", "sh_down", "sh_egate"]
    l0 = ctx.launches()
    ctx.check(ctx._lib.orn_moe_block(ctx.h, *[L[n].h for n in order], ctx.upload(x).ptr, T, k, 1, out.ptr,
                                     inds.ptr), "moe_block")
    assert ctx.launches() - l0 <= 5  # scratch index fill + the three fused kernels (13 ops unfused)
    assert np.array_equal(inds.numpy(), ref_inds)
    assert np.array_equal(out.numpy(), ref_out)
    for l in L.values():
        l.free()


def _run_worker(env_over):
    env = dict(os.environ)
    for k in ("ORN_UNFUSED", "ORN_NO_GRAPH", "ORN_NO_PDL", "ORN_PDL_MASK", "ORN_KTIME", "ORN_WIDE_EXACT",
              "ORN_NO_WIDE_PREFILL"):
        env.pop(k, None)
    env.update(env_over)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "env_worker.py")], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_control_paths_give_identical_bits():
    """ORN_UNFUSED=1 (one kernel per op), ORN_NO_GRAPH=1 (eager launches) and ORN_NO_PDL=1 (no
    programmatic dependent launch) select other execution paths of the same arithmetic: tokens,
    acceptance counts and hidden-state bits of a full-width 4-layer run and of the tiny model are
    the same in every mode."""
    base = _run_worker({})
    assert base["launches"] > 0
    for over in ({"ORN_UNFUSED": "1"}, {"ORN_NO_GRAPH": "1"}, {"ORN_NO_PDL": "1"}):
        got = _run_worker(over)
        for key in ("tiny_tokens", "tiny_stats", "full_tokens", "full_stats", "full_hidden_sha", "tiny_hidden_sha",
                    "moe_sha"):
            assert got[key] == base[key], (over, key)
    unfused = _run_worker({"ORN_UNFUSED": "1"})
    assert unfused["launches"] > 3 * base["launches"]  # really another path: one launch per op


def test_chunked_prompt_path_is_exact_with_exact_products():
    """The chunked prompt path (conv window of the chunk, KV append of T rows, causal attention
    over the chunk, the T-step recurrence, experts sorted by a counting sort and rows scattered
    back) with its products computed by the row-invariant mat-vecs (ORN_WIDE_EXACT=1) reproduces
    the 4-row windows (ORN_NO_WIDE_PREFILL=1) bit for bit: hidden rows of the prompt and the hidden
    rows of a window decoded on top of the caches it left.  With the tensor-core products the same
    path differs from it by rounding only (tests/test_gpu_prefill.py)."""
    narrow = _run_worker({"ORN_NO_WIDE_PREFILL": "1"})
    exact = _run_worker({"ORN_WIDE_EXACT": "1"})
    for key in ("tiny_prefill_sha", "tiny_after_prefill", "full_prefill_sha", "full_after_prefill"):
        assert exact[key] == narrow[key], key
    tensor = _run_worker({})
    assert tensor["tiny_prefill_sha"] != narrow["tiny_prefill_sha"]   # really another arithmetic


def test_bounded_wait_gives_up_and_the_context_survives(pkg, ctx):
    """A wait that nothing satisfies (a slot no copy was requested for) runs out of tries, the
    kernel returns, orn_sync reports ORN_ERR_TIMEOUT exactly once, and the next call works."""
    lib = ctx._lib
    ctx.sync()
    assert lib.orn_debug_wait_probe(ctx.h, 0) != 0   # argument check
    assert lib.orn_debug_wait_probe(ctx.h, 3) == 0
    rc = lib.orn_sync(ctx.h)
    assert rc == -4  # ORN_ERR_TIMEOUT
    assert b"gave up waiting" in lib.orn_last_error(ctx.h)
    assert lib.orn_sync(ctx.h) == 0   # the flag was cleared
    # ordinary work still runs and is still right
    rng = np.random.default_rng(5)
    W = hp.make_weights(rng, orc.A8, 1, 64, 256)
    x = hp.f32_to_bf16(rng.standard_normal((1, 256)).astype(np.float32))
    L = pkg.Linear.from_numpy(ctx, W.kind, W.w, W.s, W.b, E=1, O=64, K=256)
    assert np.array_equal(L.matmul(ctx.upload(x), 1).numpy(), orc.gemv(W, x, 1))
    L.free()


def test_exchange_wait_for_a_peer_gives_up_and_the_context_survives(pkg, ctx):
    """The expert-parallel exchange over peer memory waits for its peers' flags with a limit: the gather
    kernel of a group of two, with nobody playing the second rank, gives up after a few seconds, the
    status is ORN_ERR_TIMEOUT once, and the context works afterwards.  No peer, no fault, no hang."""
    import time
    lib = ctx._lib
    ctx.sync()
    t0 = time.time()
    assert lib.orn_debug_ep_wait_probe(ctx.h) == 0
    assert time.time() - t0 < 10.0
    assert lib.orn_sync(ctx.h) == -4  # ORN_ERR_TIMEOUT
    assert b"gave up waiting" in lib.orn_last_error(ctx.h)
    assert lib.orn_sync(ctx.h) == 0
    rng = np.random.default_rng(6)
    W = hp.make_weights(rng, orc.A8, 1, 64, 256)
    x = hp.f32_to_bf16(rng.standard_normal((1, 256)).astype(np.float32))
    L = pkg.Linear.from_numpy(ctx, W.kind, W.w, W.s, W.b, E=1, O=64, K=256)
    assert np.array_equal(L.matmul(ctx.upload(x), 1).numpy(), orc.gemv(W, x, 1))
    L.free()


def test_frspec_can_be_replaced_after_decoding(pkg, ctx, full4):
    """A second id list after graphs were captured: the cycle graph that drafted through the old
    pruned head is dropped and captured again (its arguments would point at freed memory)."""
    cfg, om, gm = full4
    rng = np.random.default_rng(21)
    prompt = rng.integers(0, cfg.vocab, 5).astype(np.uint32)
    c = gm.make_cache()
    ar = pkg.generate_step(gm, c, prompt, 10)
    for seed in (1, 2):
        ids = np.sort(np.random.default_rng(seed).choice(cfg.vocab, 4096 * seed, replace=False)).astype(np.uint32)
        gm.set_frspec(ids)
        L = gm.get_linear("lm_head")
        w, s, b = L.export()
        head = orc.Weights(L.kind, 1, L.O, L.K, w, s, b)
        om.set_frspec(hp.gather_rows_weights(head, ids), ids)
        ref, rst = om.generate_mtp(prompt, 1, 10, policy=1, frspec=True)
        for _ in range(3):  # eager, capture, replay
            c.reset()
            got, gst = pkg.generate_step_mtp(gm, c, prompt, 1, 10, policy=1, frspec=True)
            assert got == ar == ref
            assert (gst.cycles, gst.accepted) == (rst.cycles, rst.accepted)
    c.free()
