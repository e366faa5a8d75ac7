"""Model-level properties of the CPU oracle on a tiny model (no GPU)."""
import numpy as np
import pytest

import helpers as hp
import orn_oracle as orc


@pytest.fixture(scope="module")
def tiny():
    cfg = hp.tiny_config(orc.Config)
    W = hp.tiny_model_weights(cfg, seed=5)
    return cfg, W, orc.Model(cfg, W)


def test_forward_rows_equal_single_steps(tiny):
    """A T-row window gives each row the bits it gets stepped alone
    (tests/mtp.rs:177-234 'window vs steps')."""
    cfg, W, m = tiny
    ids = np.array([3, 77, 1500, 9, 12], np.uint32)
    c1, c2 = m.new_cache(), m.new_cache()
    a = np.concatenate([m.forward(c1, ids[i:i + 1]) for i in range(5)])
    b = np.concatenate([m.forward(c2, ids[:2]), m.forward(c2, ids[2:5])])
    assert np.array_equal(a, b)
    m.free_cache(c1)
    m.free_cache(c2)


def test_speculative_tracks_autoregressive(tiny):
    """tests/mtp.rs:246-349: MTP greedy output is the autoregressive greedy output."""
    cfg, W, m = tiny
    prompt = np.array([5, 900, 33, 1201, 8, 64, 700], np.uint32)
    ar = m.generate(prompt, 24)
    assert len(ar) == 24
    for policy in (0, 1):
        spec, st = m.generate_mtp(prompt, 1, 24, policy=policy)
        assert spec == ar
        assert st.drafted == st.cycles and st.accepted <= st.drafted
    for p in (0.5, 0.9):
        spec, st = m.generate_mtp(prompt, 1, 24, policy=1, force=(ar, p, 42))
        assert spec == ar
        assert st.accepted >= 1
    spec2, st2 = m.generate_mtp(prompt, 2, 24, policy=1, force=(ar, 0.9, 7))
    assert spec2 == ar and st2.reached_by_depth[1] >= 1


def test_frspec_cannot_change_tokens(tiny):
    """src/frspec.rs:10-16: a pruned draft head changes acceptance, never output."""
    cfg, W, m = tiny
    rng = np.random.default_rng(0)
    ids = np.sort(rng.choice(cfg.vocab, 512, replace=False)).astype(np.uint32)
    m.set_frspec(hp.gather_rows_weights(W["lm_head"], ids), ids)
    prompt = np.array([1, 2, 3, 4], np.uint32)
    ar = m.generate(prompt, 12)
    spec, _ = m.generate_mtp(prompt, 1, 12, policy=1, frspec=True, force=(ar, 0.5, 3))
    assert spec == ar
