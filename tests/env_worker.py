"""Child process of tests/test_gpu_fullwidth.py: runs fixed seeded workloads through the C ABI
under whatever ORN_* control variables the parent set and prints one JSON line with the tokens,
the acceptance counts and digests of hidden-state bits, so that the parent can compare modes."""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, HERE)
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import helpers as hp  # noqa: E402
from conftest import load_package  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def stats(st):
    return [st.cycles, st.drafted, st.accepted] + list(st.accepted_by_depth)


def main():
    pkg = load_package()
    ctx = pkg.Context(0)
    out = {}
    # tiny model: every structural feature, weights uploaded from numpy
    cfg = hp.tiny_config(pkg.Config)
    W = hp.tiny_model_weights(cfg, seed=5)
    gm = hp.upload_model(pkg, ctx, cfg, W)
    prompt = np.array([5, 900, 33, 1201, 8, 64, 700], np.uint32)
    c = gm.make_cache()
    ar = pkg.generate_step(gm, c, prompt, 20)
    c.reset()
    toks, st = pkg.generate_step_mtp(gm, c, prompt, 2, 20, force=(ar, 0.6, 4))
    out["tiny_tokens"], out["tiny_stats"] = toks, stats(st)
    c.reset()
    h = [gm.forward(c, prompt[a:b]).numpy() for a, b in [(0, 1), (1, 3), (3, 7)]]
    out["tiny_hidden_sha"] = sha(np.concatenate(h))
    # a 70-token prompt through orn_prefill (one chunk; which arithmetic it uses is the parent's choice)
    c.reset()
    long_ids = np.random.default_rng(4).integers(0, cfg.vocab, 70).astype(np.uint32)
    out["tiny_prefill_sha"] = sha(gm.prefill(c, long_ids, prefill_step=2048, want_hidden=True).numpy())
    out["tiny_after_prefill"] = sha(gm.forward(c, prompt[:2]).numpy())   # the caches it left behind
    c.free()
    gm.free()
    # full-width layers, random-init on the device
    cfg = pkg.qwen35_config(max_ctx=96, n_layers=4)
    gm = pkg.TextModel(ctx, cfg)
    gm.init_random(99)
    rng = np.random.default_rng(8)
    prompt = rng.integers(0, cfg.vocab, 7).astype(np.uint32)
    c = gm.make_cache()
    ar = pkg.generate_step(gm, c, prompt, 16)
    c.reset()
    l0 = ctx.launches()
    toks, st = pkg.generate_step_mtp(gm, c, prompt, 1, 16, force=(ar, 0.5, 4))
    out["launches"] = int(ctx.launches() - l0)
    out["full_tokens"], out["full_stats"] = toks, stats(st)
    assert toks == ar
    c.reset()
    h = [gm.forward(c, prompt[a:b]).numpy() for a, b in [(0, 2), (2, 3), (3, 7)]]
    out["full_hidden_sha"] = sha(np.concatenate(h))
    # one MoE block through orn_moe_block (fused route unless ORN_UNFUSED=1)
    order = ["gate", "switch_mlp.gate_proj", "switch_mlp.up_proj", "switch_mlp.down_proj", "shared_expert.gate_proj",
             "shared_expert.up_proj", "shared_expert.down_proj", "shared_expert_gate"]
    L = [gm.get_linear("layers.1.mlp." + n) for n in order]
    x = hp.f32_to_bf16(rng.standard_normal((2, cfg.hidden)).astype(np.float32))
    y, inds = ctx.empty((2, cfg.hidden), np.uint16), ctx.empty((2, cfg.top_k), np.uint32)
    ctx.check(ctx._lib.orn_moe_block(ctx.h, *[l.h for l in L], ctx.upload(x).ptr, 2, cfg.top_k, 1, y.ptr, inds.ptr),
              "moe_block")
    out["moe_sha"] = sha(y.numpy()) + sha(inds.numpy())
    c.reset()
    long_ids = rng.integers(0, cfg.vocab, 70).astype(np.uint32)
    out["full_prefill_sha"] = sha(gm.prefill(c, long_ids, prefill_step=2048, want_hidden=True).numpy())
    out["full_after_prefill"] = sha(gm.forward(c, prompt[:3]).numpy())
    c.free()
    gm.free()
    ctx.close()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
