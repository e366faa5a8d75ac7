"""The CPU oracle against the reference's own numpy tools (golden fixtures made
by tests/golden/make_golden.py) and against first principles."""
import os

import numpy as np
import pytest

import helpers as hp
import orn_oracle as orc

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def q4k():
    return np.load(os.path.join(G, "q4k_golden.npz"))


def test_q4k_field_packing_matches_reference(q4k):
    # tools/q4k.py put_scale_min_k4 / get_scale_min_k4
    assert np.array_equal(hp.put_scale_min_k4(q4k["sc"], q4k["mn"]), q4k["packed"])
    qs = np.zeros((64, 128), np.uint8)
    sc, mn, _ = orc.q4k_fields(qs, np.ascontiguousarray(q4k["packed"]))
    assert np.array_equal(sc, q4k["sc"]) and np.array_equal(mn, q4k["mn"])


@pytest.mark.parametrize("which", ["q", "r"])
def test_q4k_dequantize_is_bit_exact(q4k, which):
    # tools/q4k.py:98-119 (asserted equal to ggml's dequantize_row_q4_K by the reference)
    out = orc.q4k_dequantize(np.ascontiguousarray(q4k["qs_" + which]).view(np.uint8),
                             np.ascontiguousarray(q4k["scales_" + which]),
                             np.ascontiguousarray(q4k["dm_" + which]))
    assert np.array_equal(out.view(np.uint32), q4k["deq_" + which].view(np.uint32))


def test_q4k_quantizer_matches_reference(q4k):
    # the plain min/max writer used for the synthetic artifacts (tools/q4k.py:122-161)
    qs, scales, dm, _ = hp.quantize_q4k(q4k["w"])
    assert np.array_equal(qs, np.ascontiguousarray(q4k["qs_q"]).view(np.uint8).reshape(qs.shape))
    assert np.array_equal(scales, q4k["scales_q"].reshape(scales.shape))
    assert np.array_equal(dm.reshape(-1), q4k["dm_q"].reshape(-1))


def test_q4k_integer_fields_nibble_order(q4k):
    # element i and i+32 of each 64-wide group share a byte, low nibble first
    qs = np.ascontiguousarray(q4k["qs_r"]).view(np.uint8).reshape(24, 128)
    _, _, q = orc.q4k_fields(qs, np.ascontiguousarray(q4k["scales_r"]))
    for g in range(4):
        assert np.array_equal(q[:, 64 * g:64 * g + 32], qs[:, 32 * g:32 * g + 32] & 0xF)
        assert np.array_equal(q[:, 64 * g + 32:64 * g + 64], qs[:, 32 * g:32 * g + 32] >> 4)


def test_a8_layout_and_dot_match_reference():
    g = np.load(os.path.join(G, "a8_golden.npz"))
    # mlx packs four 8-bit codes per u32, lowest field first: byte i of a row is code i
    assert np.array_equal(np.ascontiguousarray(g["words"]).view(np.uint8).reshape(16, 256), g["q"])
    W = orc.Weights(orc.A8, 1, 16, 256, np.ascontiguousarray(g["words"]).view(np.uint8),
                    hp.f32_to_bf16(g["scales"]), hp.f32_to_bf16(g["biases"]))
    # stored scales/biases are already bfloat16 values
    assert np.array_equal(hp.bf16_to_f32(W.s), g["scales"]) and np.array_equal(hp.bf16_to_f32(W.b), g["biases"])
    rng = np.random.default_rng(1)
    x = hp.f32_to_bf16(rng.standard_normal(256).astype(np.float32))
    y = orc.gemv(W, x, 1, f32=True)[0]
    ref = g["deq"].astype(np.float64) @ hp.bf16_to_f32(x).astype(np.float64)
    assert np.max(hp.rel_err(y, ref)) < 2e-4 or np.max(np.abs(y - ref)) < 1e-5
    # quantiser used for the synthetic artifacts reconstructs as well as mlx's
    q, s, b = hp.quantize_a8(g["w"])
    mine = (hp.bf16_to_f32(s)[:, None] * q + hp.bf16_to_f32(b)[:, None]).reshape(16, 256)
    assert np.abs(mine - g["w"]).max() <= 1.5 * np.abs(g["deq"] - g["w"]).max() + 1e-6


def test_a4_layout_and_dot_match_reference():
    """mlx affine 4-bit group 32 as tools/aq.py states it: eight codes per u32, lowest nibble
    first; the oracle's mat-vec on that layout against the tool's dequantised weights; the
    synthetic-weight quantiser is the tool's, bit for bit."""
    g = np.load(os.path.join(G, "a4_golden.npz"))
    by = np.ascontiguousarray(g["words"]).view(np.uint8).reshape(16, 128)
    assert np.array_equal(by & 0xF, g["q"][:, 0::2]) and np.array_equal(by >> 4, g["q"][:, 1::2])
    q, s, b = hp.quantize_affine(g["w"], 32, 4)
    assert np.array_equal(q.reshape(16, 256), g["q"])
    assert np.array_equal(hp.bf16_to_f32(s).reshape(16, 8), g["scales"]) and np.array_equal(hp.bf16_to_f32(b).reshape(16, 8), g["biases"])
    assert np.array_equal(hp.pack_nibbles(q).reshape(16, 128), by)
    W = orc.Weights(orc.A4, 1, 16, 256, by, hp.f32_to_bf16(g["scales"]), hp.f32_to_bf16(g["biases"]))
    rng = np.random.default_rng(2)
    x = hp.f32_to_bf16(rng.standard_normal(256).astype(np.float32))
    y = orc.gemv(W, x, 1, f32=True)[0]
    ref = g["deq"].astype(np.float64) @ hp.bf16_to_f32(x).astype(np.float64)
    assert np.max(hp.rel_err(y, ref)) < 2e-4 or np.max(np.abs(y - ref)) < 1e-5


def test_byte_model_matches_the_reference_accounting():
    """bench.py's algorithmic bytes per token against the reference's own tool (tools/step_bytes.py
    run on header-only artifacts of the full-size model, tests/golden/make_golden.py): the
    benchmark's mix, and the published q6k-full mix whose 1.8051 GB the reference documents."""
    import json
    import sys
    ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, ROOT)
    import bench
    gold = json.load(open(os.path.join(G, "step_bytes_golden.json")))
    assert abs(gold["published"]["total_gb"] - 1.8051) < 5e-5
    cfg = bench.qwen35_dims(40, 512)
    mine = bench.step_bytes(cfg, 1, with_state=False) / 1e9
    assert abs(mine - gold["benchmark"]["total_gb"]) / gold["benchmark"]["total_gb"] < 1e-3, (mine, gold["benchmark"])
    # the inventory the fixtures were made from reproduces both totals with the tool's rules
    size = {"BF16": 2, "F16": 2, "U32": 4, "U8": 1, "I8": 1}
    for mix in ("benchmark", "published"):
        total = 0
        for name, (dt, shape) in hp.artifact_inventory(cfg, mix).items():
            n = int(np.prod(shape)) * size[dt]
            if ".switch_mlp." in name:
                n = n * cfg.top_k // cfg.n_experts
            elif "embed_tokens" in name:
                n //= cfg.vocab
            total += n
        assert abs(total / 1e9 - gold[mix]["total_gb"]) < 1e-4, (mix, total)


def test_bf16_rounding_matches_reference():
    g = np.load(os.path.join(G, "bf16_golden.npz"))
    assert np.array_equal(hp.bf16_to_f32(hp.f32_to_bf16(g["x"])).view(np.uint32), g["r"].view(np.uint32))
    # src/array.rs:272-276: ties go to even
    assert hp.f32_to_bf16(np.array([1.00390625], np.float32))[0] == 0x3F80
    assert hp.f32_to_bf16(np.array([1.01171875], np.float32))[0] == 0x3F82


def test_frspec_id_file_is_the_reference_tools(tmp_path):
    """The id file the reference's tools/merge_frspec.py writes (fixture: 300 ids with duplicates, which
    the tool sorts and dedupes): u32 count, then the ids, little endian.  The writer the GPU loader tests
    use produces the same bytes for the same list, so `orn_frspec_load` is tested on the tool's format."""
    g = np.load(os.path.join(G, "frspec_ids_golden.npz"))
    want = np.unique(g["ids_in"]).astype(np.uint32)
    raw = g["file_bytes"].tobytes()
    assert int(g["n"]) == len(want)
    assert np.frombuffer(raw[:4], "<u4")[0] == len(want)
    assert np.array_equal(np.frombuffer(raw[4:], "<u4"), want)
    cfg = hp.tiny_config(orc.Config)
    d = hp.write_artifact(str(tmp_path / "art"), cfg, hp.tiny_model_weights(cfg, seed=1), frspec_ids=want % cfg.vocab)
    mine = open(os.path.join(d, "ids.bin"), "rb").read()
    assert mine[:4] == raw[:4] and len(mine) == len(raw)
    assert np.array_equal(np.frombuffer(mine[4:], "<u4"), want % cfg.vocab)


def test_q6k_artifact_layout_is_the_reference_split():
    """Raw 210-byte Q6_K blocks cut into artifact tensors by the reference's own tools/q4k.py split
    (fixture): ql|qh in one tensor, int8 sub-block scales, one float16 d per block.  The oracle reading
    those tensors gives what ggml's published dequantize_row_q6_K gives on the raw blocks (ql at byte 0,
    qh at 128, scales at 192, d at 208), restated here in numpy on the BLOCK form."""
    g = np.load(os.path.join(G, "q6k_golden.npz"))
    blocks = g["blocks"]                                    # [48, 210]
    qs = np.ascontiguousarray(g["qs"]).view(np.uint8)       # [24, 2 * 192]
    assert np.array_equal(qs.reshape(48, 192), blocks[:, :192])
    assert np.array_equal(g["scales"].reshape(48, 16), blocks[:, 192:208])
    assert np.array_equal(g["dm"].reshape(48), np.ascontiguousarray(blocks[:, 208:210]).view(np.uint16).reshape(48))
    out = orc.q6k_dequantize(np.ascontiguousarray(qs), np.ascontiguousarray(g["scales"]).view(np.int8),
                             np.ascontiguousarray(g["dm"]))
    ql, qh = blocks[:, 0:128].astype(np.int32), blocks[:, 128:192].astype(np.int32)
    sc = np.ascontiguousarray(blocks[:, 192:208]).view(np.int8).astype(np.float32)
    d = np.ascontiguousarray(blocks[:, 208:210]).view(np.float16).astype(np.float32)[:, 0]
    ref = np.zeros((48, 256), np.float32)
    for n in range(2):            # the two 128-weight halves of a block
        for l in range(32):
            a, b_, h = ql[:, 64 * n + l], ql[:, 64 * n + l + 32], qh[:, 32 * n + l]
            codes = ((a & 0xF) | ((h & 3) << 4), (b_ & 0xF) | (((h >> 2) & 3) << 4),
                     (a >> 4) | (((h >> 4) & 3) << 4), (b_ >> 4) | (((h >> 6) & 3) << 4))
            for c, q in enumerate(codes):
                ref[:, 128 * n + 32 * c + l] = d * sc[:, 8 * n + l // 16 + 2 * c] * (q - 32)
    assert np.array_equal(out.reshape(48, 256).view(np.uint32), ref.view(np.uint32))


def test_q6k_dequantize_formula():
    # kernels/q6k.metal:47-77 restated independently in numpy
    rng = np.random.default_rng(3)
    W = hp.raw_q6k(rng, 1, 4, 512)
    out = orc.q6k_dequantize(W.w, W.s.view(np.int8), W.b)
    w = W.w.reshape(-1, 192)
    ql, qh = w[:, :128].astype(np.int32), w[:, 128:].astype(np.int32)
    sc = W.s.view(np.int8).reshape(-1, 16).astype(np.float32)
    d = W.b.view(np.float16).astype(np.float32).reshape(-1, 1)
    ref = np.zeros((len(w), 256), np.float32)
    for n in range(2):
        for l in range(32):
            is_ = l // 16
            a, b_, h = ql[:, 64 * n + l], ql[:, 64 * n + l + 32], qh[:, 32 * n + l]
            q1 = ((a & 0xF) | ((h & 3) << 4)) - 32
            q2 = ((b_ & 0xF) | (((h >> 2) & 3) << 4)) - 32
            q3 = ((a >> 4) | (((h >> 4) & 3) << 4)) - 32
            q4 = ((b_ >> 4) | (((h >> 6) & 3) << 4)) - 32
            for c, q in enumerate((q1, q2, q3, q4)):
                ref[:, 128 * n + 32 * c + l] = d[:, 0] * sc[:, 8 * n + is_ + 2 * c] * q
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))
    # the round-to-nearest writer used for synthetic artifacts round-trips
    wf = (rng.standard_normal((8, 256)) * 0.02).astype(np.float32)
    q, s, dd = hp.quantize_q6k(wf)
    back = orc.q6k_dequantize(q, s.view(np.int8), dd)
    assert np.abs(back - wf).max() < 0.02 * 4 / 31


@pytest.mark.parametrize("kind,K", [(orc.Q4K, 2048), (orc.Q6K, 512), (orc.Q6K, 2048), (orc.A8, 2048),
                                    (orc.A8, 4096), (orc.BF16, 2048), (orc.Q4K, 256)])
def test_gemv_matches_float64_dot(kind, K):
    """Config-1 shape: the dot within 1e-4 relative of the float64 dot of the
    dequantised weights (tests/q4k.rs:337-388 uses the same statement)."""
    rng = np.random.default_rng(K + kind)
    O = 64
    W = {orc.Q4K: hp.raw_q4k, orc.Q6K: hp.raw_q6k}.get(kind, None)
    W = W(rng, 1, O, K) if W else hp.make_weights(rng, kind, 1, O, K)
    x = hp.f32_to_bf16(rng.standard_normal(K).astype(np.float32))
    y = orc.gemv(W, x, 1, f32=True)[0]
    if kind == orc.Q4K:
        deq = orc.q4k_dequantize(W.w, W.s, W.b).reshape(O, K)
    elif kind == orc.Q6K:
        deq = orc.q6k_dequantize(W.w, W.s.view(np.int8), W.b).reshape(O, K)
    elif kind == orc.A8:
        deq = (hp.bf16_to_f32(W.s).reshape(O, -1, 1) * W.w.reshape(O, -1, 64)
               + hp.bf16_to_f32(W.b).reshape(O, -1, 1)).reshape(O, K)
    else:
        deq = hp.bf16_to_f32(W.w).reshape(O, K)
    ref = deq.astype(np.float64) @ hp.bf16_to_f32(x).astype(np.float64)
    scale = np.abs(deq.astype(np.float64)) @ np.abs(hp.bf16_to_f32(x).astype(np.float64))
    assert np.max(np.abs(y - ref) / scale) < 1e-5
    assert np.median(hp.rel_err(y, ref)) < 1e-4


def test_gemv_one_hot_returns_a_column():
    # tests/q4k.rs:85-107: a one-hot activation returns a dequantised column
    rng = np.random.default_rng(7)
    W = hp.raw_q4k(rng, 1, 16, 512)
    deq = orc.q4k_dequantize(W.w, W.s, W.b).reshape(16, 512)
    for col in (0, 31, 32, 255, 300, 511):
        x = np.zeros(512, np.float32)
        x[col] = 1.0
        y = orc.gemv(W, hp.f32_to_bf16(x), 1, f32=True)[0]
        assert np.max(hp.rel_err(y, deq[:, col])) < 1e-6


def test_gemv_rows_are_batch_invariant():
    # tests/batch_invariance.rs:85-232: row r of an M-row call == the row alone
    rng = np.random.default_rng(11)
    for kind in (orc.Q4K, orc.Q6K, orc.A8, orc.BF16):
        W = hp.make_weights(rng, kind, 1, 32, 512)
        x = hp.f32_to_bf16(rng.standard_normal((4, 512)).astype(np.float32))
        y4 = orc.gemv(W, x, 4)
        for r in range(4):
            assert np.array_equal(orc.gemv(W, x[r], 1)[0], y4[r])
        z = orc.gemv(W, np.zeros((1, 512), np.uint16), 1, f32=True)
        assert np.all(z == 0.0)  # a zero row gives exact zeros (tests/q4k.rs:238-269)


def test_router_topk_tie_rule():
    # kernels/moe.metal:568-614: by value, then by larger index; ascending slots
    g = np.zeros((1, 16), np.float32)
    g[0, [2, 5, 9]] = 0.25
    g[0, 7] = 0.5
    gates = hp.f32_to_bf16(g)
    inds, scores = orc.router_topk(gates, 1, 16, 4)
    assert inds[0].tolist() == [2, 5, 9, 7]
    assert hp.bf16_to_f32(scores)[0].tolist() == [0.25, 0.25, 0.25, 0.5]
    # all equal: the k largest indices, ascending
    inds, _ = orc.router_topk(hp.f32_to_bf16(np.full((1, 16), 0.0625, np.float32)), 1, 16, 4)
    assert inds[0].tolist() == [12, 13, 14, 15]


def test_greedy_lowest_index_on_ties_and_lse():
    rng = np.random.default_rng(5)
    V = 5000
    x = rng.standard_normal(V).astype(np.float32)
    x[[100, 4000]] = 7.0
    lg = hp.f32_to_bf16(x)
    assert orc.greedy_token(lg, True) == 100 and orc.greedy_token(lg, False) == 100
    lse = hp.bf16_to_f32(np.array([orc.logsumexp(lg)], np.uint16))[0]
    xs = hp.bf16_to_f32(lg).astype(np.float64)
    ref = np.log(np.sum(np.exp(xs - xs.max()))) + xs.max()
    assert abs(lse - ref) <= abs(ref) * 2 ** -8


def test_sigmoid_and_softplus_tables_against_float64():
    """Every bfloat16 input (tests/activations.rs does the same against mlx)."""
    import ctypes as C
    lib = orc.lib()
    # the oracle has no exported scalar entry points; go through sigmoid_gate / gdn paths
    h = np.arange(0, 65536, dtype=np.uint32).astype(np.uint16)
    x = hp.bf16_to_f32(h)
    ok = np.isfinite(x)
    ones = hp.f32_to_bf16(np.ones(ok.sum(), np.float32))
    got = hp.bf16_to_f32(orc.sigmoid_gate(np.ascontiguousarray(h[ok]), ones, int(ok.sum()), 1))
    xd = x[ok].astype(np.float64)
    e = hp.bf16_to_f32(hp.f32_to_bf16(np.exp(np.minimum(np.abs(xd), 89.0)).astype(np.float32))).astype(np.float64)
    d = hp.bf16_to_f32(hp.f32_to_bf16((1.0 + e).astype(np.float32))).astype(np.float64)
    y = hp.bf16_to_f32(hp.f32_to_bf16((1.0 / d).astype(np.float32))).astype(np.float64)
    ref = np.where(xd < 0, y, hp.bf16_to_f32(hp.f32_to_bf16((1.0 - y).astype(np.float32))))
    bad = np.flatnonzero(got != ref.astype(np.float32))
    # the exponential is ~1 ulp, so a handful of inputs may sit on a bfloat16 rounding boundary
    assert len(bad) <= 8, (len(bad), x[ok][bad][:8])
    assert np.max(np.abs(got - ref)) <= 2 ** -8
