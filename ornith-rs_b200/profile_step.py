"""Small profiling driver: a 4-layer model with the real layer sizes (one
3:1 gated-delta/attention period, 256 experts, full vocabulary; ~3.3 GB on the
device) running a few MTP depth-1 cycles.  Meant to sit under `ncu`, where the
full 40-layer benchmark is too large to capture.

    python ornith-rs_b200/profile_step.py [tokens]
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import __graft_entry__ as ge  # noqa: E402


def main():
    tokens = int(sys.argv[1]) if len(sys.argv) > 1 else 8
    pkg = ge.load_package()
    ctx = pkg.Context(0)
    cfg = pkg.qwen35_config(max_ctx=128, n_layers=4)
    m = pkg.TextModel(ctx, cfg)
    m.init_random(1)
    c = m.make_cache()
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, 5).astype(np.uint32)
    ar = pkg.generate_step(m, c, prompt, tokens)
    c.reset()
    got, st = pkg.generate_step_mtp(m, c, prompt, 1, tokens, force=(ar, 0.5, 1))
    assert got == ar
    p = m.prof()
    print("tokens %d cycles %d decode %.3f ms launches %d" % (len(got), st.cycles, p.total_ms, p.kernel_launches))


if __name__ == "__main__":
    main()
