"""CUDA kernels against the CPU oracle through the C ABI, bit for bit."""
import numpy as np
import pytest

import helpers as hp
import orn_oracle as orc

pytestmark = pytest.mark.gpu


def lin_of(pkg, ctx, W):
    return pkg.Linear.from_numpy(ctx, W.kind, W.w, W.s, W.b, E=W.E, O=W.O, K=W.K)


def bf(rng, shape, scale=1.0):
    return hp.f32_to_bf16((rng.standard_normal(shape) * scale).astype(np.float32))


def test_config1_q4k_matvec(pkg, ctx):
    """BASELINE config 1: N=512 x K=2048 raw-field Q4_K, x ~ N(0,1) bf16, fp32 out."""
    rng = np.random.default_rng(1)
    W = hp.raw_q4k(rng, 1, 512, 2048)
    x = bf(rng, 2048)
    L = lin_of(pkg, ctx, W)
    # integer dequant: bit-exact
    deq = L.dequantize().numpy()
    ref = orc.q4k_dequantize(W.w, W.s, W.b).reshape(512, 2048)
    assert np.array_equal(deq.view(np.uint32), ref.view(np.uint32))
    # dot: bit-exact against the oracle, and within 1e-4 relative of float64
    y = L.matmul(ctx.upload(x), 1, out_f32=True).numpy()[0]
    assert np.array_equal(y.view(np.uint32), orc.gemv(W, x, 1, f32=True)[0].view(np.uint32))
    r64 = ref.astype(np.float64) @ hp.bf16_to_f32(x).astype(np.float64)
    mag = np.abs(ref.astype(np.float64)) @ np.abs(hp.bf16_to_f32(x).astype(np.float64))
    assert np.max(np.abs(y - r64) / mag) < 1e-5
    assert np.median(hp.rel_err(y, r64)) < 1e-4


@pytest.mark.parametrize("kind", [orc.Q4K, orc.Q6K, orc.A8, orc.BF16, orc.A4])
@pytest.mark.parametrize("O,K", [(37, 512), (100, 2048), (256, 4096), (1, 2048), (64, 256)])
def test_gemv_bit_exact_all_widths(pkg, ctx, kind, O, K):
    rng = np.random.default_rng(O * 7 + K + kind)
    raw = {orc.Q4K: hp.raw_q4k, orc.Q6K: hp.raw_q6k}.get(kind)
    W = raw(rng, 1, O, K) if (raw and O % 2) else hp.make_weights(rng, kind, 1, O, K)
    L = lin_of(pkg, ctx, W)
    x = bf(rng, (5, K))
    xd = ctx.upload(x)
    for M in (1, 2, 3, 4, 5):
        got = L.matmul(xd, M).numpy()
        assert np.array_equal(got, orc.gemv(W, x[:M], M)), (kind, O, K, M)
    if kind in (orc.Q4K, orc.Q6K):
        deq = L.dequantize().numpy()
        ref = (orc.q4k_dequantize(W.w, W.s, W.b) if kind == orc.Q4K
               else orc.q6k_dequantize(W.w, W.s.view(np.int8), W.b)).reshape(O, K)
        assert np.array_equal(deq.view(np.uint32), ref.view(np.uint32))
    # export gives back the artifact tensors
    w, s, b = L.export()
    assert np.array_equal(w, W.w.reshape(-1).view(np.uint8))
    if W.s is not None:
        assert np.array_equal(s, W.s.reshape(-1).view(np.uint8)) and np.array_equal(b, W.b.reshape(-1).view(np.uint8))
    L.free()


@pytest.mark.parametrize("kind,O,K", [(orc.Q4K, 512, 2048), (orc.Q6K, 2048, 512), (orc.BF16, 64, 512), (orc.A8, 40, 256),
                                       (orc.A4, 48, 512)])
def test_gather_gemv(pkg, ctx, kind, O, K):
    """Routed rows: 11 rows over 4 experts, unsorted (tools/dump_q4k.py:177-199 shapes)."""
    rng = np.random.default_rng(kind + 3)
    W = hp.make_weights(rng, kind, 4, O, K)
    L = lin_of(pkg, ctx, W)
    x = bf(rng, (3, K))
    lhs = np.array([0, 1, 2, 0, 1, 2, 2, 1, 0, 0, 1], np.uint32)
    rhs = np.array([3, 0, 1, 2, 2, 3, 0, 1, 0, 3, 3], np.uint32)
    got = L.gather_matmul(ctx.upload(x), ctx.upload(lhs), ctx.upload(rhs), 11).numpy()
    assert np.array_equal(got, orc.gather_gemv(W, x, lhs, rhs))
    L.free()


def test_random_init_matches_oracle_decode(pkg, ctx):
    """Weights generated on the GPU, exported, and fed to the oracle."""
    rng = np.random.default_rng(2)
    for kind, O, K in [(orc.Q4K, 48, 512), (orc.Q6K, 48, 512), (orc.A8, 48, 512), (orc.BF16, 48, 512)]:
        L = pkg.Linear.random(ctx, kind, 2, O, K, seed=1234 + kind)
        w, s, b = L.export()
        W = orc.Weights(kind, 2, O, K, w, s if s.size else None, b if b.size else None)
        x = bf(rng, (2, K))
        lhs = np.array([0, 1, 1], np.uint32)
        rhs = np.array([1, 0, 1], np.uint32)
        got = L.gather_matmul(ctx.upload(x), ctx.upload(lhs), ctx.upload(rhs), 3).numpy()
        assert np.array_equal(got, orc.gather_gemv(W, x, lhs, rhs))
        # N(0, 0.02)-like weights
        if kind == orc.Q4K:
            d = orc.q4k_dequantize(w, s, b)
            assert 0.015 < d.std() < 0.025 and abs(d.mean()) < 2e-3
        L.free()


def test_embedding(pkg, ctx):
    rng = np.random.default_rng(4)
    W = hp.make_weights(rng, orc.A8, 1, 300, 512)
    L = lin_of(pkg, ctx, W)
    ids = np.array([0, 299, 17, 17], np.uint32)
    out = ctx.empty((4, 512), np.uint16)
    ctx.check(ctx._lib.orn_embedding(ctx.h, L.h, ctx.upload(ids).ptr, 4, out.ptr), "embedding")
    assert np.array_equal(out.numpy(), orc.embedding(W, ids))


@pytest.mark.parametrize("rows,n", [(1, 2048), (7, 2048), (16, 128), (5, 256), (3, 512)])
def test_norms(pkg, ctx, rows, n):
    rng = np.random.default_rng(rows + n)
    a, b, z = bf(rng, (rows, n), 3.0), bf(rng, (rows, n)), bf(rng, (rows, n))
    w = hp.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(n).astype(np.float32))
    eps = 1e-6
    o = ctx.empty((rows, n), np.uint16)
    ctx.check(ctx._lib.orn_rms_norm(ctx.h, ctx.upload(a).ptr, ctx.upload(w).ptr, rows, n, eps, o.ptr), "rms")
    assert np.array_equal(o.numpy(), orc.rms_norm(a, w, rows, n, eps))
    ctx.check(ctx._lib.orn_rms_norm(ctx.h, ctx.upload(a).ptr, None, rows, n, eps, o.ptr), "rms")
    assert np.array_equal(o.numpy(), orc.rms_norm(a, None, rows, n, eps))
    h = ctx.empty((rows, n), np.uint16)
    ctx.check(ctx._lib.orn_add_rms_norm(ctx.h, ctx.upload(a).ptr, ctx.upload(b).ptr, ctx.upload(w).ptr, rows, n,
                                        eps, h.ptr, o.ptr), "add_rms")
    rh, ro = orc.add_rms_norm(a, b, w, rows, n, eps)
    assert np.array_equal(h.numpy(), rh) and np.array_equal(o.numpy(), ro)
    ctx.check(ctx._lib.orn_rms_norm_gated(ctx.h, ctx.upload(a).ptr, ctx.upload(w).ptr, ctx.upload(z).ptr, rows, n,
                                          eps, o.ptr), "gated")
    assert np.array_equal(o.numpy(), orc.rms_norm_gated(a, w, z, rows, n, eps))


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("kinds", [(orc.A8,), (orc.A8, orc.A8, orc.BF16, orc.BF16), (orc.Q4K, orc.A8), (orc.BF16,),
                                   (orc.Q6K, orc.A8), (orc.Q4K, orc.Q6K, orc.A8, orc.BF16)])
def test_fused_add_norm_gemv(pkg, ctx, M, kinds):
    """The persistent norm + mat-vec kernel equals add_rms_norm then gemv, bit for bit."""
    if len(kinds) == 4 and len(set(kinds)) == 4 and M > 2:
        pytest.skip("four staged copies of more than two rows do not fit shared memory; no model mixes four formats")
    rng = np.random.default_rng(100 * M + len(kinds) + kinds[0])
    K, eps = 2048, 1e-6
    Os = [300, 37, 32, 1][:len(kinds)]
    a, b = bf(rng, (M, K), 2.0), bf(rng, (M, K))
    w = hp.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(K).astype(np.float32))
    Ws = [hp.make_weights(rng, kind, 1, O, K) for kind, O in zip(kinds, Os)]
    Ls = [lin_of(pkg, ctx, W) for W in Ws]
    for second in (b, None):
        outs, h, normed = pkg.add_norm_gemv(ctx, ctx.upload(a), ctx.upload(second) if second is not None else None,
                                            ctx.upload(w), M, K, eps, Ls, want_h=True, want_normed=True)
        if second is not None:
            rh, rx = orc.add_rms_norm(a, second, w, M, K, eps)
            assert np.array_equal(h.numpy(), rh)
        else:
            rx = orc.rms_norm(a, w, M, K, eps)
        assert np.array_equal(normed.numpy(), rx)
        for W, o in zip(Ws, outs):
            assert np.array_equal(o.numpy(), orc.gemv(W, rx, M)), (W.kind, M)
    for L in Ls:
        L.free()


def test_elementwise_every_bf16_input(pkg, ctx):
    """sigmoid_gate and swiglu over all 65536 bfloat16 inputs (tests/activations.rs)."""
    h = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    rng = np.random.default_rng(9)
    other = bf(rng, 65536)
    o = ctx.empty((65536,), np.uint16)
    notnan = ~np.isnan(hp.bf16_to_f32(h))  # NaN payloads are not part of the contract
    ctx.check(ctx._lib.orn_sigmoid_gate(ctx.h, ctx.upload(h).ptr, ctx.upload(other).ptr, 65536, 1, o.ptr), "sg")
    assert np.array_equal(o.numpy()[notnan], orc.sigmoid_gate(h, other, 65536, 1)[notnan])
    ctx.check(ctx._lib.orn_swiglu(ctx.h, ctx.upload(h).ptr, ctx.upload(other).ptr, 65536, o.ptr), "swiglu")
    got, ref = o.numpy()[notnan], orc.swiglu(h, other)[notnan]
    gnan, rnan = np.isnan(hp.bf16_to_f32(got)), np.isnan(hp.bf16_to_f32(ref))  # silu(-inf) = -inf * 0
    assert np.array_equal(gnan, rnan) and np.array_equal(got[~gnan], ref[~rnan])
    # host copies of the shared elementary functions equal the device ones
    x = hp.bf16_to_f32(h)
    fin = np.isfinite(x)
    lib = pkg.lib()
    host = np.array([lib.orn_host_sigmoid_bf(float(v)) for v in x[fin][::97]], np.float32)
    ones = hp.f32_to_bf16(np.ones(65536, np.float32))
    ctx.check(ctx._lib.orn_sigmoid_gate(ctx.h, ctx.upload(h).ptr, ctx.upload(ones).ptr, 65536, 1, o.ptr), "sg")
    assert np.array_equal(hp.bf16_to_f32(o.numpy())[fin][::97], host)


@pytest.mark.parametrize("T", [1, 2, 7, 40])   # 40: the combine's eight-columns-per-thread form (16 rows and more)
def test_router_softmax_topk_combine(pkg, ctx, T):
    rng = np.random.default_rng(T)
    n, k, dim = 256, 8, 2048
    logits = bf(rng, (T, n), 2.0)
    logits[0, 5] = logits[0, 200]  # an exact tie
    p = ctx.empty((T, n), np.uint16)
    ctx.check(ctx._lib.orn_softmax_precise(ctx.h, ctx.upload(logits).ptr, T, n, p.ptr), "softmax")
    rp = orc.softmax_precise(logits, T, n)
    assert np.array_equal(p.numpy(), rp)
    inds, scores = ctx.empty((T, k), np.uint32), ctx.empty((T, k), np.uint16)
    ctx.check(ctx._lib.orn_router_topk(ctx.h, p.ptr, T, n, k, inds.ptr, scores.ptr), "topk")
    ri, rs = orc.router_topk(rp, T, n, k)
    assert np.array_equal(inds.numpy(), ri) and np.array_equal(scores.numpy(), rs)
    y, gate, shared = bf(rng, (T, k, dim)), bf(rng, (T,)), bf(rng, (T, dim))
    out = ctx.empty((T, dim), np.uint16)
    for norm in (1, 0):
        ctx.check(ctx._lib.orn_moe_combine(ctx.h, scores.ptr, ctx.upload(y).ptr, ctx.upload(gate).ptr,
                                           ctx.upload(shared).ptr, T, k, dim, norm, out.ptr), "combine")
        assert np.array_equal(out.numpy(), orc.moe_combine(rs, y, gate, shared, T, k, dim, norm))


@pytest.mark.parametrize("T", [1, 2])
def test_config2_moe_layer(pkg, ctx, T):
    """BASELINE config 2 at reduced expert count for the CPU side: hidden 2048,
    router N(0,0.02), experts Q4_K gate/up [512,2048], Q6_K down [2048,512],
    shared expert of the same shapes with a sigmoid gate; inds bit-exact."""
    rng = np.random.default_rng(20 + T)
    H, E, I, k = 2048, 32, 512, 8
    ws = {
        "gate": hp.make_weights(rng, orc.BF16, 1, E, H),
        "sw_gate": hp.raw_q4k(rng, E, I, H), "sw_up": hp.raw_q4k(rng, E, I, H),
        "sw_down": hp.raw_q6k(rng, E, H, I),
        "sh_gate": hp.raw_q4k(rng, 1, I, H), "sh_up": hp.raw_q4k(rng, 1, I, H),
        "sh_down": hp.raw_q6k(rng, 1, H, I), "sh_egate": hp.make_weights(rng, orc.A8, 1, 1, H),
    }
    x = bf(rng, (T, H))
    ref_out, ref_inds = orc.moe_block(ws, x, T, k, 1)
    L = {n: lin_of(pkg, ctx, w) for n, w in ws.items()}
    out, inds = ctx.empty((T, H), np.uint16), ctx.empty((T, k), np.uint32)
    order = ["gate", "sw_gate", "sw_up", "sw_down", "sh_gate", "sh_up", "sh_down", "sh_egate"]
    ctx.check(ctx._lib.orn_moe_block(ctx.h, *[L[n].h for n in order], ctx.upload(x).ptr, T, k, 1, out.ptr,
                                     inds.ptr), "moe_block")
    assert np.array_equal(inds.numpy(), ref_inds)
    assert np.array_equal(out.numpy(), ref_out)
    for l in L.values():
        l.free()


def gdn_inputs(rng, T, Hk=16, Hv=32, Dh=128, Kc=4):
    D = 2 * Hk * Dh + Hv * Dh
    return dict(conv_state=bf(rng, (Kc - 1, D), 0.5), qkv=bf(rng, (T, D)), cw=bf(rng, (D, Kc), 0.2),
                a=bf(rng, (T, Hv)), b=bf(rng, (T, Hv)), a_log=bf(rng, (Hv,), 0.3), dt_bias=bf(rng, (Hv,), 0.3))


def run_front(ctx, i, T, Hk, Hv, Dh, Kc):
    D = 2 * Hk * Dh + Hv * Dh
    o = dict(conv_next=ctx.empty((Kc - 1, D), np.uint16), q=ctx.empty((T, Hk, Dh), np.uint16),
             k=ctx.empty((T, Hk, Dh), np.uint16), v=ctx.empty((T, Hv, Dh), np.uint16),
             beta=ctx.empty((T, Hv), np.uint16), g=ctx.empty((T, Hv), np.float32))
    d = {n: ctx.upload(v) for n, v in i.items()}
    ctx.check(ctx._lib.orn_gdn_front(ctx.h, d["conv_state"].ptr, d["qkv"].ptr, d["cw"].ptr, d["a"].ptr, d["b"].ptr,
                                     d["a_log"].ptr, d["dt_bias"].ptr, T, Hk, Hv, Dh, Kc, 1e-6, o["conv_next"].ptr,
                                     o["q"].ptr, o["k"].ptr, o["v"].ptr, o["beta"].ptr, o["g"].ptr), "gdn_front")
    return o


@pytest.mark.parametrize("T", [1, 2, 7])
def test_config3_gdn_layer(pkg, ctx, T):
    """BASELINE config 3: 16 key / 32 value heads of 128, conv k=4, zero or
    non-zero fp32 state; decode, verify (+rollback) and a short prefill."""
    rng = np.random.default_rng(30 + T)
    Hk, Hv, Dh, Kc = 16, 32, 128, 4
    i = gdn_inputs(rng, T)
    ref = orc.gdn_front(i["conv_state"], i["qkv"], i["cw"], i["a"], i["b"], i["a_log"], i["dt_bias"], T, Hk, Hv, Dh, Kc)
    o = run_front(ctx, i, T, Hk, Hv, Dh, Kc)
    for name, r in zip(["conv_next", "q", "k", "v", "beta"], ref[:5]):
        assert np.array_equal(o[name].numpy(), r), name
    assert np.array_equal(o["g"].numpy().view(np.uint32), ref[5].view(np.uint32))
    for init in ("zero", "random"):
        st0 = np.zeros((Hv, 128, 128), np.float32) if init == "zero" else \
            (0.1 * rng.standard_normal((Hv, 128, 128))).astype(np.float32)
        st_ref = st0.copy()
        y_ref, snaps_ref = orc.gated_delta(ref[1], ref[2], ref[3], ref[5], ref[4], st_ref, T, Hk, Hv, want_snaps=True)
        st = ctx.upload(st0)
        snaps = ctx.empty((T, Hv, 128, 128), np.float32)
        y = ctx.empty((T, Hv, 128), np.uint16)
        ctx.check(ctx._lib.orn_gated_delta(ctx.h, o["q"].ptr, o["k"].ptr, o["v"].ptr, o["g"].ptr, o["beta"].ptr,
                                           st.ptr, T, Hk, Hv, y.ptr, snaps.ptr), "gated_delta")
        assert np.array_equal(y.numpy(), y_ref)
        assert np.array_equal(st.numpy().view(np.uint32), st_ref.view(np.uint32))
        assert np.array_equal(snaps.numpy().view(np.uint32), snaps_ref.view(np.uint32))
        # rollback to keep=1: snapshot 0 is exactly the state a T=1 call leaves
        st1 = ctx.upload(st0)
        y1 = ctx.empty((1, Hv, 128), np.uint16)
        ctx.check(ctx._lib.orn_gated_delta(ctx.h, o["q"].ptr, o["k"].ptr, o["v"].ptr, o["g"].ptr, o["beta"].ptr,
                                           st1.ptr, 1, Hk, Hv, y1.ptr, None), "gated_delta")
        assert np.array_equal(st1.numpy().view(np.uint32), snaps_ref[0].view(np.uint32))
        assert np.array_equal(y1.numpy()[0], y_ref[0])


def test_config3_gdn_prefill_6621(pkg, ctx):
    """T = 6621 through the same sequential kernels; checked against the oracle
    on a prefix and by chunk-invariance for the whole length."""
    rng = np.random.default_rng(33)
    Hk, Hv, Dh, Kc, T = 16, 32, 128, 4, 6621
    i = gdn_inputs(rng, T)
    o = run_front(ctx, i, T, Hk, Hv, Dh, Kc)
    Tp = 96
    ref = orc.gdn_front(i["conv_state"], i["qkv"][:Tp], i["cw"], i["a"][:Tp], i["b"][:Tp], i["a_log"], i["dt_bias"],
                        Tp, Hk, Hv, Dh, Kc)
    assert np.array_equal(o["q"].numpy()[:Tp], ref[1]) and np.array_equal(o["v"].numpy()[:Tp], ref[3])
    st_ref = np.zeros((Hv, 128, 128), np.float32)
    y_ref = orc.gated_delta(ref[1], ref[2], ref[3], ref[5], ref[4], st_ref, Tp, Hk, Hv)
    # one call over the full length
    st = ctx.zeros((Hv, 128, 128), np.float32)
    y = ctx.empty((T, Hv, 128), np.uint16)
    ctx.check(ctx._lib.orn_gated_delta(ctx.h, o["q"].ptr, o["k"].ptr, o["v"].ptr, o["g"].ptr, o["beta"].ptr, st.ptr,
                                       T, Hk, Hv, y.ptr, None), "gated_delta")
    yh = y.numpy()
    assert np.array_equal(yh[:Tp], y_ref)
    # chunks of 2048 (the reference's prefill step) give the same bits
    st2 = ctx.zeros((Hv, 128, 128), np.float32)
    y2 = ctx.empty((T, Hv, 128), np.uint16)
    for t0 in range(0, T, 2048):
        n = min(2048, T - t0)
        ctx.check(ctx._lib.orn_gated_delta(
            ctx.h, o["q"].at(t0 * Hk * 128 * 2), o["k"].at(t0 * Hk * 128 * 2), o["v"].at(t0 * Hv * 128 * 2),
            o["g"].at(t0 * Hv * 4), o["beta"].at(t0 * Hv * 2), st2.ptr, n, Hk, Hv, y2.at(t0 * Hv * 128 * 2), None),
            "gated_delta")
    assert np.array_equal(y2.numpy(), yh)
    assert np.array_equal(st2.numpy().view(np.uint32), st.numpy().view(np.uint32))
    assert np.isfinite(st.numpy()).all()


@pytest.mark.parametrize("T,init", [(64, "zero"), (100, "random"), (37, "random"), (6621, "zero"), (2048, "random")])
def test_gated_delta_chunkwise_agrees_with_the_sequential_kernel(pkg, ctx, T, init):
    """The prompt path's chunkwise recurrence (64-token chunks on the warp tensor cores) against
    orn_gated_delta (bit-equal to the oracle above) at BASELINE config 3's head counts: outputs and
    the final state.  bf16 operands with f32 accumulation: the rms of the difference is held below
    1 % of the rms of the values (0.25 % expected), the largest difference below 6 % of the largest value."""
    rng = np.random.default_rng(500 + T)
    Hk, Hv, Dh, Kc = 16, 32, 128, 4
    i = gdn_inputs(rng, T)
    o = run_front(ctx, i, T, Hk, Hv, Dh, Kc)
    st0 = np.zeros((Hv, 128, 128), np.float32) if init == "zero" else \
        (0.1 * rng.standard_normal((Hv, 128, 128))).astype(np.float32)
    outs = []
    for fn in ("orn_gated_delta", "orn_gated_delta_prefill"):
        st = ctx.upload(st0)
        y = ctx.empty((T, Hv, 128), np.uint16)
        args = [ctx.h, o["q"].ptr, o["k"].ptr, o["v"].ptr, o["g"].ptr, o["beta"].ptr, st.ptr, T, Hk, Hv, y.ptr]
        if fn == "orn_gated_delta":
            args.append(None)
        ctx.check(getattr(ctx._lib, fn)(*args), fn)
        outs.append((hp.bf16_to_f32(y.numpy()).astype(np.float64), st.numpy().astype(np.float64)))
    (yw, sw), (yg, sg) = outs
    assert np.isfinite(yg).all() and np.isfinite(sg).all()
    for want, got, what in ((yw, yg, "y"), (sw, sg, "state")):
        rms = np.sqrt((want ** 2).mean())
        assert np.sqrt(((want - got) ** 2).mean()) <= 1e-2 * rms, (what, np.sqrt(((want - got) ** 2).mean()) / rms)
        assert np.abs(want - got).max() <= 6e-2 * np.abs(want).max(), (what, np.abs(want - got).max() / np.abs(want).max())


@pytest.mark.parametrize("T,offset", [(1, 0), (1, 37), (4, 0), (2, 4095)])
def test_rope(pkg, ctx, T, offset):
    rng = np.random.default_rng(T + offset)
    x = bf(rng, (T, 16, 256))
    d = ctx.upload(x)
    ctx.check(ctx._lib.orn_rope(ctx.h, d.ptr, T, 16, 256, 64, 1e7, offset), "rope")
    assert np.array_equal(d.numpy(), orc.rope(x, T, 16, 256, 64, 1e7, offset))


@pytest.mark.parametrize("T,Lk", [(1, 512), (1, 2048), (4, 4), (2, 53), (1, 1), (3, 100)])
def test_sdpa_decode(pkg, ctx, T, Lk):
    """Shapes of tools/dump_attn.py:47-52 at 16/2 heads x 256; causal inside the window."""
    rng = np.random.default_rng(T * 1000 + Lk)
    Hq, Hkv, hd, cap = 16, 2, 256, max(Lk, 64)
    offset = Lk - T
    q = bf(rng, (T, Hq, hd))
    kc, vc = bf(rng, (Hkv, cap, hd)), bf(rng, (Hkv, cap, hd))
    out = ctx.empty((T, Hq, hd), np.uint16)
    ctx.check(ctx._lib.orn_sdpa_decode(ctx.h, ctx.upload(q).ptr, ctx.upload(kc).ptr, ctx.upload(vc).ptr, T, Hq, Hkv,
                                       hd, cap, offset, 1.0 / 16.0, out.ptr), "sdpa")
    ref = orc.sdpa_decode(q, kc, vc, T, Hq, Hkv, hd, cap, offset, 1.0 / 16.0)
    got = out.numpy()
    assert np.array_equal(got, ref)
    # row r of the window equals the same token stepped alone
    one = ctx.empty((1, Hq, hd), np.uint16)
    for r in range(T):
        ctx.check(ctx._lib.orn_sdpa_decode(ctx.h, ctx.upload(q[r:r + 1]).ptr, ctx.upload(kc).ptr, ctx.upload(vc).ptr,
                                           1, Hq, Hkv, hd, cap, offset + r, 1.0 / 16.0, one.ptr), "sdpa")
        assert np.array_equal(one.numpy()[0], got[r])


@pytest.mark.parametrize("T,offset", [(64, 0), (100, 0), (37, 300), (200, 1000), (1, 5), (130, 31)])
def test_sdpa_prefill_agrees_with_the_row_invariant_kernel(pkg, ctx, T, offset):
    """The prompt path's tensor-core attention against orn_sdpa_decode (itself bit-equal to the
    oracle above): same contract, another summation order and bf16 probabilities.  Tolerance: an
    output is a convex combination of V entries (|v| up to about 4 here), so 2e-2 absolute is a few
    bf16 steps of the largest term; the mean error is checked an order of magnitude tighter."""
    rng = np.random.default_rng(T * 7 + offset)
    Hq, Hkv, hd = 16, 2, 256
    cap = offset + T + 9
    q = bf(rng, (T, Hq, hd))
    kc, vc = bf(rng, (Hkv, cap, hd)), bf(rng, (Hkv, cap, hd))
    dq, dk, dv = ctx.upload(q), ctx.upload(kc), ctx.upload(vc)
    want, got = ctx.empty((T, Hq, hd), np.uint16), ctx.empty((T, Hq, hd), np.uint16)
    for r in range(0, T, 4):          # the row-invariant kernel takes windows of up to 4 rows
        n = min(4, T - r)
        ctx.check(ctx._lib.orn_sdpa_decode(ctx.h, dq.at(r * Hq * hd * 2), dk.ptr, dv.ptr, n, Hq, Hkv, hd, cap, offset + r,
                                           1.0 / 16.0, want.at(r * Hq * hd * 2)), "sdpa")
    ctx.check(ctx._lib.orn_sdpa_prefill(ctx.h, dq.ptr, dk.ptr, dv.ptr, T, Hq, Hkv, hd, cap, offset, 1.0 / 16.0, got.ptr),
              "sdpa_prefill")
    w, g = hp.bf16_to_f32(want.numpy()).astype(np.float64), hp.bf16_to_f32(got.numpy()).astype(np.float64)
    assert np.isfinite(g).all()
    assert np.abs(w - g).max() < 2e-2, np.abs(w - g).max()
    assert np.abs(w - g).mean() < 2e-3, np.abs(w - g).mean()


@pytest.mark.parametrize("V", [248320, 1000, 1024, 5000])
def test_greedy(pkg, ctx, V):
    rng = np.random.default_rng(V)
    T = 3
    x = (rng.standard_normal((T, V)) * 1.5).astype(np.float32)
    x[0, [V // 3, V - 1]] = 9.0           # tie at the maximum: lowest index wins
    x[1, V - 7] = 8.0
    x[1, 11] = 7.96875                   # one bf16 step below: merges after the subtraction or not
    lg = hp.f32_to_bf16(x)
    d = ctx.upload(lg)
    for norm in (1, 0):
        toks = ctx.empty((T,), np.uint32)
        ctx.check(ctx._lib.orn_greedy(ctx.h, d.ptr, T, V, norm, toks.ptr), "greedy")
        ref = [orc.greedy_token(lg[t], norm) for t in range(T)]
        assert toks.numpy().tolist() == ref
    assert ref[0] == V // 3


def test_errors_are_reported_not_fatal(pkg, ctx):
    lib = ctx._lib
    import ctypes as C
    h = C.c_void_p()
    w = np.zeros(16, np.uint8)
    assert lib.orn_linear_create(ctx.h, orc.Q4K, 1, 4, 100, w.ctypes.data, w.ctypes.data, w.ctypes.data, C.byref(h)) == -1
    assert b"multiple of 256" in lib.orn_last_error(ctx.h)
    assert lib.orn_gemv(ctx.h, None, None, 1, None, 0) == -1
    x = ctx.zeros((16,), np.uint16)
    assert lib.orn_sdpa_decode(ctx.h, x.ptr, x.ptr, x.ptr, 1, 16, 2, 128, 64, 0, 1.0, x.ptr) == -1
    ctx.sync()  # the context is still usable
