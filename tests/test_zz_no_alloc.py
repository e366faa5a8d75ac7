"""orn_greedy_static (greedy sampling on the library's fixed device scratch, no
allocation) against orn_greedy and the oracle, through the C ABI.  The file name
sorts last so that the default collection order runs it after every other test;
it also passes on its own."""
import numpy as np
import pytest

import helpers as hp
import orn_oracle as orc

pytestmark = pytest.mark.gpu


def _logits(seed, T, V):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((T, V)) * 1.5).astype(np.float32)
    x[0, [V // 3, V - 1]] = 9.0  # a tie at the maximum: the lowest index wins
    if T > 1:
        x[1, V - 7] = 8.0
        x[1, 11] = 7.96875       # one bfloat16 step below the maximum
    return hp.f32_to_bf16(x)


@pytest.mark.parametrize("T,V", [(1, 1000), (3, 5000), (4, 248320), (2, 262144), (2, 1025)])
def test_static_greedy_equals_allocating_greedy_twice_in_a_row(pkg, ctx, T, V):
    lib = ctx._lib
    for call in range(2):  # two calls in a row on fresh inputs: the shared scratch carries nothing over
        lg = _logits(17 * T + V + call, T, V)
        d = ctx.upload(lg)
        for norm in (1, 0):
            want = ctx.empty((T,), np.uint32)
            ctx.check(lib.orn_greedy(ctx.h, d.ptr, T, V, norm, want.ptr), "orn_greedy")
            got = ctx.empty((T,), np.uint32)
            got.set(np.full(T, 0xFFFFFFFF, np.uint32))
            ctx.check(lib.orn_greedy_static(ctx.h, d.ptr, T, V, norm, got.ptr), "orn_greedy_static")
            ctx.sync()
            assert got.numpy().tolist() == want.numpy().tolist()
            if V <= 5000:
                assert got.numpy().tolist() == [orc.greedy_token(lg[t], norm) for t in range(T)]
        d.free()


def test_static_greedy_back_to_back_without_sync(pkg, ctx):
    """Calls queued on one stream without a wait in between reuse the scratch in order."""
    lib = ctx._lib
    V = 40000
    inputs = [_logits(900 + i, 4, V) for i in range(3)]
    devs = [ctx.upload(x) for x in inputs]
    outs = [ctx.empty((4,), np.uint32) for _ in inputs]
    for d, o in zip(devs, outs):
        ctx.check(lib.orn_greedy_static(ctx.h, d.ptr, 4, V, 1, o.ptr), "orn_greedy_static")
    ctx.sync()
    for x, d, o in zip(inputs, devs, outs):
        want = ctx.empty((4,), np.uint32)
        ctx.check(lib.orn_greedy(ctx.h, d.ptr, 4, V, 1, want.ptr), "orn_greedy")
        assert o.numpy().tolist() == want.numpy().tolist()


def test_static_greedy_rejects_what_does_not_fit(pkg, ctx):
    lib = ctx._lib
    d = ctx.upload(np.zeros((1, 1024), np.uint16))
    o = ctx.empty((8,), np.uint32)
    assert lib.orn_greedy_static(ctx.h, d.ptr, 5, 128, 1, o.ptr) != 0          # more than 4 rows
    assert lib.orn_greedy_static(ctx.h, d.ptr, 1, 262145, 1, o.ptr) != 0       # more than 262144 logits
    assert lib.orn_greedy_static(ctx.h, None, 1, 1024, 1, o.ptr) != 0
    with pytest.raises(pkg.OrnError, match="orn_greedy_static"):
        ctx.check(lib.orn_greedy_static(ctx.h, d.ptr, 5, 128, 1, o.ptr), "orn_greedy_static")
    # the context stays usable
    ctx.check(lib.orn_greedy_static(ctx.h, d.ptr, 1, 1024, 1, o.ptr), "orn_greedy_static")
    ctx.sync()
    assert int(o.numpy()[0]) == 0
