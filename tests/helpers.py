"""Seeded synthetic inputs for the tests: bfloat16 helpers, the three
quantisers, raw-field generators and a tiny model in the artifact layout."""
import numpy as np

import orn_oracle as orc

Q4K, Q6K, A8, BF16, A4 = 0, 1, 2, 3, 4


# ------------------------------------------------------------------ bfloat16
def f32_to_bf16(x):
    """Round to nearest even, as src/array.rs:229-237."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_to_f32(h):
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.abs(a - b) / np.maximum(np.abs(b), 1e-30)


# ------------------------------------------------------------------ Q4_K
def put_scale_min_k4(sc, mn):
    """8 six-bit scales + 8 mins -> 12 bytes (inverse of get_scale_min_k4)."""
    sc = np.asarray(sc, np.uint8)
    mn = np.asarray(mn, np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), np.uint8)
    for j in range(4):
        out[..., j] = sc[..., j] & 63
        out[..., j + 4] = mn[..., j] & 63
    for j in range(4, 8):
        out[..., j + 4] = (sc[..., j] & 0xF) | ((mn[..., j] & 0xF) << 4)
        out[..., j - 4] |= (sc[..., j] >> 4) << 6
        out[..., j] |= (mn[..., j] >> 4) << 6
    return out


def raw_q4k(rng, E, O, K):
    """Raw-field Q4_K as in the single mat-vec benchmark config: d, dmin =
    f16(|N(0,1)| 1e-3), scales/mins uniform 0..63, uniform nibbles."""
    nb = K // 256
    n = E * O * nb
    dm = (np.abs(rng.standard_normal((n, 2))) * 1e-3).astype(np.float16)
    sc = rng.integers(0, 64, (n, 8)).astype(np.uint8)
    mn = rng.integers(0, 64, (n, 8)).astype(np.uint8)
    scales = put_scale_min_k4(sc, mn)
    qs = rng.integers(0, 256, (n, 128)).astype(np.uint8)
    return orc.Weights(Q4K, E, O, K, qs, scales, dm.view(np.uint16))


def raw_q6k(rng, E, O, K):
    nb = K // 256
    n = E * O * nb
    d = (np.abs(rng.standard_normal(n)) * 1e-3).astype(np.float16)
    scales = rng.integers(-128, 128, (n, 16)).astype(np.int8)
    w = rng.integers(0, 256, (n, 192)).astype(np.uint8)
    return orc.Weights(Q6K, E, O, K, w, scales.view(np.uint8), d.view(np.uint16))


def quantize_q4k(w):
    """Plain min/max Q4_K writer (the shape of ggml's quantize_row_q4_K_ref as
    restated in the reference's tools/q4k.py:122-161)."""
    w = np.asarray(w, np.float32)
    E_O = w.shape[:-1]
    K = w.shape[-1]
    x = w.reshape(-1, 256)
    g = x.reshape(-1, 8, 32)
    lo = np.minimum(g.min(-1), 0.0)
    hi = g.max(-1)
    scale = (hi - lo) / 15.0
    mn = -lo
    d = (scale.max(-1, keepdims=True) / 63.0).astype(np.float16).astype(np.float32)
    dm = (mn.max(-1, keepdims=True) / 63.0).astype(np.float16).astype(np.float32)
    sc = np.where(d > 0, np.clip(np.rint(scale / np.where(d > 0, d, 1)), 0, 63), 0)
    m = np.where(dm > 0, np.clip(np.rint(mn / np.where(dm > 0, dm, 1)), 0, 63), 0)
    ds, ms = d * sc, dm * m
    q = np.clip(np.rint((g + ms[..., None]) / np.where(ds > 0, ds, 1)[..., None]), 0, 15)
    q = np.where((ds > 0)[..., None], q, 0).astype(np.uint8).reshape(-1, 256)
    qs = np.empty((len(x), 128), np.uint8)
    for h in range(4):
        qs[:, 32 * h:32 * h + 32] = q[:, 64 * h:64 * h + 32] | (q[:, 64 * h + 32:64 * h + 64] << 4)
    scales = put_scale_min_k4(sc.astype(np.uint8), m.astype(np.uint8))
    dmh = np.concatenate([d, dm], -1).astype(np.float16)
    return qs, scales, dmh.view(np.uint16), (E_O, K)


def quantize_q6k(w):
    """Round-to-nearest Q6_K: 16 sub-blocks of 16, signed int8 sub-scales."""
    w = np.asarray(w, np.float32)
    x = w.reshape(-1, 256)
    g = x.reshape(-1, 16, 16)
    sub = np.abs(g).max(-1) / 31.0
    d = (sub.max(-1, keepdims=True) / 127.0).astype(np.float16).astype(np.float32)
    sc = np.where(d > 0, np.clip(np.rint(sub / np.where(d > 0, d, 1)), 1, 127), 0).astype(np.int8)
    ds = d * sc
    q = np.where((ds > 0)[..., None], np.clip(np.rint(g / np.where(ds > 0, ds, 1)[..., None]), -32, 31), 0)
    q = (q + 32).astype(np.uint8).reshape(-1, 256)
    ql = np.zeros((len(x), 128), np.uint8)
    qh = np.zeros((len(x), 64), np.uint8)
    for n in range(2):
        for c in range(4):
            v = q[:, 128 * n + 32 * c:128 * n + 32 * c + 32]
            lo4, hi2 = v & 0xF, v >> 4
            base = 64 * n + (32 if (c & 1) else 0)
            if c < 2:
                ql[:, base:base + 32] |= lo4
            else:
                ql[:, base:base + 32] |= lo4 << 4
            qh[:, 32 * n:32 * n + 32] |= hi2 << (2 * c)
    return np.concatenate([ql, qh], 1), sc.view(np.uint8), d.astype(np.float16).view(np.uint16)


def quantize_a8(w):
    """mlx affine quantise, 8 bits, group 64 (the rule restated in the
    reference's tools/aq.py:34-72): scale = (max-min)/255, bias = min."""
    w = np.asarray(w, np.float32)
    g = w.reshape(-1, 64)
    lo, hi = g.min(-1), g.max(-1)
    scale = np.maximum((hi - lo) / 255.0, 1e-8)
    sb = f32_to_bf16(scale)
    bb = f32_to_bf16(lo)
    s, b = bf16_to_f32(sb), bf16_to_f32(bb)
    q = np.clip(np.rint((g - b[:, None]) / s[:, None]), 0, 255).astype(np.uint8)
    return q, sb, bb


def quantize_affine(w, group, bits):
    """mlx's affine_quantize as the reference's tools/aq.py:34-72 restates it (scale signed towards
    the larger edge, the edge code exact, codes computed against the unrounded scale and bias,
    Metal's round half away from zero), then bfloat16 scales and biases."""
    f = np.float32
    n_bins = f((1 << bits) - 1)
    g = np.asarray(w, np.float32).reshape(-1, group)
    w_min = g.min(1)
    w_max = np.maximum(g.max(1), f(0))
    scale = np.maximum((w_max - w_min) / n_bins, f(1e-7)).astype(np.float32)
    side = np.abs(w_min) > np.abs(w_max)
    scale = np.where(side, scale, -scale).astype(np.float32)
    edge = np.where(side, w_min, w_max).astype(np.float32)
    rnd = lambda x: (np.sign(x) * np.floor(np.abs(x) + f(0.5))).astype(np.float32)
    q0 = rnd(edge / scale)
    at_zero = q0 == f(0)
    scale = np.where(at_zero, scale, edge / np.where(at_zero, f(1), q0)).astype(np.float32)
    bias = np.where(at_zero, f(0), edge).astype(np.float32)
    q = np.minimum(rnd((g - bias[:, None]) / scale[:, None]), n_bins)
    return q.astype(np.uint8), f32_to_bf16(scale), f32_to_bf16(bias)


def pack_nibbles(q):
    """4-bit codes, eight per u32 with the lowest-order field first (tools/aq.py:78-93): byte b of
    a row holds code 2b in its low nibble and code 2b+1 in its high nibble."""
    q = np.asarray(q, np.uint8).reshape(-1, 2)
    return (q[:, 0] | (q[:, 1] << 4)).astype(np.uint8)


def make_weights(rng, kind, E, O, K, std=0.02):
    w = (rng.standard_normal((E * O, K)) * std).astype(np.float32)
    if kind == Q4K:
        qs, scales, dm, _ = quantize_q4k(w)
        return orc.Weights(Q4K, E, O, K, qs, scales, dm)
    if kind == Q6K:
        q, sc, d = quantize_q6k(w)
        return orc.Weights(Q6K, E, O, K, q, sc, d)
    if kind == A8:
        q, s, b = quantize_a8(w)
        return orc.Weights(A8, E, O, K, q, s, b)
    if kind == A4:
        q, s, b = quantize_affine(w, 32, 4)
        return orc.Weights(A4, E, O, K, pack_nibbles(q).reshape(E * O, K // 2), s, b)
    return orc.Weights(BF16, E, O, K, f32_to_bf16(w))


# ------------------------------------------------------------------ tiny model
def tiny_config(cfg_cls, **over):
    """A small model with every structural feature of the 35B-A3B: three
    gated-delta layers per full-attention layer, GQA, a routed MoE with a
    shared expert, an MTP head."""
    d = dict(hidden=512, n_layers=4, full_attn_interval=4, n_heads=4, n_kv_heads=2, head_dim=256,
             rope_dims=64, rope_theta=1e7, gdn_k_heads=2, gdn_v_heads=4, gdn_head_dim=128,
             gdn_conv_kernel=4, n_experts=16, top_k=4, expert_inter=256, shared_inter=256,
             norm_topk_prob=1, vocab=1536, rms_eps=1e-6, max_ctx=96)
    d.update(over)
    return cfg_cls(**d)


def tiny_model_weights(cfg, seed=0, mix="benchmark"):
    """name -> Weights | uint16 tensor.  mix "benchmark": expert gate/up Q4_K, expert down Q6_K,
    everything else 8-bit affine, MTP head bf16.  mix "published": the module formats of the
    reference's q6k-full artifact (tools/forge_q4k.py:131-152): gated-delta projections, lm_head and
    routed experts Q4_K, attention projections and routers Q6_K, shared experts affine 4-bit group
    32, embedding and shared-expert gate 8-bit affine."""
    rng = np.random.default_rng(seed)
    pub = mix == "published"
    LIN, ATT, HEAD = (Q4K, Q6K, Q4K) if pub else (A8, A8, A8)
    H = cfg.hidden
    D = 2 * cfg.gdn_k_heads * cfg.gdn_head_dim + cfg.gdn_v_heads * cfg.gdn_head_dim
    VD = cfg.gdn_v_heads * cfg.gdn_head_dim
    QD, KVD = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    W = {}

    def ten(name, n, mean, std):
        W[name] = f32_to_bf16(mean + std * rng.standard_normal(n).astype(np.float32))

    def moe(p, dense):
        q4, q6, a8 = (BF16, BF16, BF16) if dense else (Q4K, Q6K, A8)
        router, down, sh = (a8, q6, None) if (dense or not pub) else (Q6K, Q4K, A4)
        W[p + "gate"] = make_weights(rng, router, 1, cfg.n_experts, H)
        W[p + "switch_mlp.gate_proj"] = make_weights(rng, q4, cfg.n_experts, cfg.expert_inter, H)
        W[p + "switch_mlp.up_proj"] = make_weights(rng, q4, cfg.n_experts, cfg.expert_inter, H)
        W[p + "switch_mlp.down_proj"] = make_weights(rng, down, cfg.n_experts, H, cfg.expert_inter)
        W[p + "shared_expert.gate_proj"] = make_weights(rng, sh if sh is not None else q4, 1, cfg.shared_inter, H)
        W[p + "shared_expert.up_proj"] = make_weights(rng, sh if sh is not None else q4, 1, cfg.shared_inter, H)
        W[p + "shared_expert.down_proj"] = make_weights(rng, sh if sh is not None else q6, 1, H, cfg.shared_inter)
        W[p + "shared_expert_gate"] = make_weights(rng, a8, 1, 1, H)

    W["embed_tokens"] = make_weights(rng, A8, 1, cfg.vocab, H)
    W["lm_head"] = make_weights(rng, HEAD, 1, cfg.vocab, H)
    ten("norm.weight", H, 1.0, 0.05)
    for i in range(cfg.n_layers):
        lp = "layers.%d." % i
        ten(lp + "input_layernorm.weight", H, 1.0, 0.05)
        ten(lp + "post_attention_layernorm.weight", H, 1.0, 0.05)
        if (i + 1) % cfg.full_attn_interval != 0:
            a = lp + "linear_attn."
            W[a + "in_proj_qkv"] = make_weights(rng, LIN, 1, D, H)
            W[a + "in_proj_z"] = make_weights(rng, LIN, 1, VD, H)
            W[a + "in_proj_a.weight"] = make_weights(rng, BF16, 1, cfg.gdn_v_heads, H)
            W[a + "in_proj_b.weight"] = make_weights(rng, BF16, 1, cfg.gdn_v_heads, H)
            W[a + "out_proj"] = make_weights(rng, LIN, 1, H, VD)
            ten(a + "conv1d.weight", D * cfg.gdn_conv_kernel, 0.0, 0.2)
            ten(a + "dt_bias", cfg.gdn_v_heads, 0.0, 0.3)
            ten(a + "A_log", cfg.gdn_v_heads, 0.0, 0.3)
            ten(a + "norm.weight", cfg.gdn_head_dim, 1.0, 0.05)
        else:
            a = lp + "self_attn."
            W[a + "q_proj"] = make_weights(rng, ATT, 1, 2 * QD, H)
            W[a + "k_proj"] = make_weights(rng, ATT, 1, KVD, H)
            W[a + "v_proj"] = make_weights(rng, ATT, 1, KVD, H)
            W[a + "o_proj"] = make_weights(rng, ATT, 1, H, QD)
            ten(a + "q_norm.weight", cfg.head_dim, 1.0, 0.05)
            ten(a + "k_norm.weight", cfg.head_dim, 1.0, 0.05)
        moe(lp + "mlp.", False)
    lp = "mtp.layers.0."
    ten("mtp.pre_fc_norm_embedding.weight", H, 1.0, 0.05)
    ten("mtp.pre_fc_norm_hidden.weight", H, 1.0, 0.05)
    W["mtp.fc.weight"] = make_weights(rng, BF16, 1, H, 2 * H)
    ten("mtp.norm.weight", H, 1.0, 0.05)
    ten(lp + "input_layernorm.weight", H, 1.0, 0.05)
    ten(lp + "post_attention_layernorm.weight", H, 1.0, 0.05)
    W[lp + "self_attn.q_proj.weight"] = make_weights(rng, BF16, 1, 2 * QD, H)
    W[lp + "self_attn.k_proj.weight"] = make_weights(rng, BF16, 1, KVD, H)
    W[lp + "self_attn.v_proj.weight"] = make_weights(rng, BF16, 1, KVD, H)
    W[lp + "self_attn.o_proj.weight"] = make_weights(rng, BF16, 1, H, QD)
    ten(lp + "self_attn.q_norm.weight", cfg.head_dim, 1.0, 0.05)
    ten(lp + "self_attn.k_norm.weight", cfg.head_dim, 1.0, 0.05)
    moe(lp + "mlp.", True)
    return W


def gather_rows_weights(W, ids):
    """FrSpec::prune on host tensors (row gather of every head tensor)."""
    ids = np.asarray(ids)
    rw = W.w.reshape(W.O, -1)[ids]
    rs = None if W.s is None else W.s.reshape(W.O, -1)[ids]
    rb = None if W.b is None else W.b.reshape(W.O, -1)[ids]
    return orc.Weights(W.kind, 1, len(ids), W.K, rw, rs, rb)


def upload_model(pkg, ctx, cfg, weights):
    """Register the same tensors with the CUDA library."""
    m = pkg.TextModel(ctx, cfg)
    for name, w in weights.items():
        if isinstance(w, orc.Weights):
            lin = pkg.Linear.from_numpy(ctx, w.kind, w.w, w.s, w.b, E=w.E, O=w.O, K=w.K)
            m.set_linear(name, lin)
        else:
            m.set_tensor(name, w)
    return m


# ---------------------------------------------------------------------------
# a seeded artifact on disk in the reference's layout (src/safetensors.rs:189-308,
# src/weights.rs:179-279, tools/forge_q4k.py:40-48): config.json, sharded
# safetensors with an index, the MTP sidecar with numbered experts, FR-Spec ids
# ---------------------------------------------------------------------------
def _st_write(path, tensors):
    """tensors: name -> (dtype string, shape, bytes)."""
    import json
    header, off, blobs = {}, 0, []
    for name, (dt, shape, raw) in tensors.items():
        header[name] = {"dtype": dt, "shape": [int(x) for x in shape], "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(len(hj).to_bytes(8, "little"))
        f.write(hj)
        for b in blobs:
            f.write(b)


def _module_tensors(name, W):
    """The artifact tensors of one weight module."""
    import orn_oracle as orc
    lead = [W.E] if W.E > 1 else []
    raw = lambda a: np.ascontiguousarray(a).tobytes()
    nb = W.K // 256
    if W.kind == orc.Q4K:
        return {name + ".weight": ("U32", lead + [W.O, W.K // 8], raw(W.w)),
                name + ".scales": ("U8", lead + [W.O, nb, 12], raw(W.s)),
                name + ".dm": ("F16", lead + [W.O, nb, 2], raw(W.b))}
    if W.kind == orc.Q6K:
        return {name + ".weight": ("U32", lead + [W.O, 3 * W.K // 16], raw(W.w)),
                name + ".scales": ("I8", lead + [W.O, nb, 16], raw(W.s)),
                name + ".dm": ("F16", lead + [W.O, nb, 1], raw(W.b))}
    if W.kind == orc.A8:
        return {name + ".weight": ("U32", lead + [W.O, W.K // 4], raw(W.w)),
                name + ".scales": ("BF16", lead + [W.O, W.K // 64], raw(W.s)),
                name + ".biases": ("BF16", lead + [W.O, W.K // 64], raw(W.b))}
    if W.kind == orc.A4:
        return {name + ".weight": ("U32", lead + [W.O, W.K // 8], raw(W.w)),
                name + ".scales": ("BF16", lead + [W.O, W.K // 32], raw(W.s)),
                name + ".biases": ("BF16", lead + [W.O, W.K // 32], raw(W.b))}
    return None


QUANT_SPEC = {0: {"mode": "q4k", "group_size": 256, "bits": 4}, 1: {"mode": "q6k", "group_size": 256, "bits": 6},
              2: {"mode": "affine", "group_size": 64, "bits": 8}, 4: {"mode": "affine", "group_size": 32, "bits": 4}}


def write_artifact(directory, cfg, W, frspec_ids=None, quant_block=False):
    """Writes the tiny model as the reference stores a model on disk; returns the directory.
    quant_block: config.json carries the per-module `quantization` table of a published artifact
    (default affine 4-bit group 32, an override per module in another mode, src/weights.rs:49-79)."""
    import json
    import os
    import orn_oracle as orc
    os.makedirs(os.path.join(directory, "mtp"), exist_ok=True)
    text = {"hidden_size": cfg.hidden, "num_hidden_layers": cfg.n_layers, "num_attention_heads": cfg.n_heads,
            "num_key_value_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
            "full_attention_interval": cfg.full_attn_interval,
            "rope_parameters": {"rope_theta": cfg.rope_theta, "partial_rotary_factor": cfg.rope_dims / cfg.head_dim},
            "linear_num_key_heads": cfg.gdn_k_heads, "linear_num_value_heads": cfg.gdn_v_heads,
            "linear_key_head_dim": cfg.gdn_head_dim, "linear_value_head_dim": cfg.gdn_head_dim,
            "linear_conv_kernel_dim": cfg.gdn_conv_kernel, "num_experts": cfg.n_experts,
            "num_experts_per_tok": cfg.top_k, "moe_intermediate_size": cfg.expert_inter,
            "shared_expert_intermediate_size": cfg.shared_inter, "norm_topk_prob": bool(cfg.norm_topk_prob),
            "vocab_size": cfg.vocab, "rms_norm_eps": cfg.rms_eps}
    top = {"model_type": "qwen3_5_moe", "text_config": text,
           "mlx_lm_extra_tensors": {"mtp_file": "mtp/weights.safetensors"}}
    if quant_block:
        qb = {"group_size": 32, "bits": 4, "mode": "affine"}
        for name, w in W.items():
            if isinstance(w, orc.Weights) and w.kind in QUANT_SPEC and w.kind != orc.A4:
                full = name if name.startswith("mtp.") else (
                    "language_model.lm_head" if name == "lm_head" else "language_model.model." + name)
                qb[full[:-len(".weight")] if full.endswith(".weight") else full] = QUANT_SPEC[w.kind]
        top["quantization"] = qb
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(top, f)
    trunk, side = {}, {}
    for name, w in W.items():
        is_mtp = name.startswith("mtp.")
        dst = side if is_mtp else trunk
        full = name if is_mtp else ("language_model.lm_head" if name == "lm_head" else "language_model.model." + name)
        if isinstance(w, orc.Weights):
            mod = full[:-len(".weight")] if full.endswith(".weight") else full
            t = _module_tensors(mod, w)
            if t is not None:
                dst.update(t)
            elif w.E > 1:  # bf16 experts of the MTP head: numbered, one matrix each (src/weights.rs:237-279)
                proj = mod.rsplit(".", 1)[1]
                base = mod[:-len("switch_mlp." + proj)] + "experts."
                per = w.w.reshape(w.E, w.O, w.K)
                for e in range(w.E):
                    dst["%s%d.%s.weight" % (base, e, proj)] = ("BF16", [w.O, w.K], per[e].tobytes())
            else:
                dst[mod + ".weight"] = ("BF16", [w.O, w.K], np.ascontiguousarray(w.w).tobytes())
        else:
            dst[full] = ("BF16", list(np.shape(w)), np.ascontiguousarray(w).tobytes())
    # two shards + index, as a published artifact has
    names = sorted(trunk)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for fn, ns in shards.items():
        _st_write(os.path.join(directory, fn), {n: trunk[n] for n in ns})
        weight_map.update({n: fn for n in ns})
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    _st_write(os.path.join(directory, "mtp", "weights.safetensors"), side)
    if frspec_ids is not None:  # u32 count then the ids, little endian (src/frspec.rs:67-148)
        ids = np.ascontiguousarray(frspec_ids, np.uint32)
        with open(os.path.join(directory, "ids.bin"), "wb") as f:
            f.write(np.uint32(len(ids)).tobytes())
            f.write(ids.tobytes())
    return directory


# ---------------------------------------------------------------------------
# tensor inventory of a full-size artifact (names, dtypes, shapes; no data): what
# tools/step_bytes.py of the reference reads from the safetensors headers
# ---------------------------------------------------------------------------
def artifact_inventory(cfg, mix):
    """name -> (dtype, shape) of every trunk tensor.  mix "benchmark": BASELINE config 4 (expert
    gate/up Q4_K, expert down Q6_K, the rest 8-bit affine group 64).  mix "published": the
    reference's q6k-full artifact (tools/forge_q4k.py:24-35,131-152): layers 0..31 keep their routed
    experts in Q4_K and their shared experts in affine 4-bit group 32, layers 32..39 hold both in
    Q6_K; gated-delta projections and lm_head Q4_K; attention projections and routers Q6_K;
    embedding and shared-expert gates 8-bit affine."""
    H, V, E, I, SI = cfg.hidden, cfg.vocab, cfg.n_experts, cfg.expert_inter, cfg.shared_inter
    D = 2 * cfg.gdn_k_heads * cfg.gdn_head_dim + cfg.gdn_v_heads * cfg.gdn_head_dim
    VD, QD, KVD = cfg.gdn_v_heads * cfg.gdn_head_dim, cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    inv = {}

    def mod(name, kind, O, K, lead=()):
        lead = list(lead)
        nb = K // 256
        if kind == Q4K:
            inv[name + ".weight"] = ("U32", lead + [O, K // 8])
            inv[name + ".scales"] = ("U8", lead + [O, nb, 12])
            inv[name + ".dm"] = ("F16", lead + [O, nb, 2])
        elif kind == Q6K:
            inv[name + ".weight"] = ("U32", lead + [O, 3 * K // 16])
            inv[name + ".scales"] = ("I8", lead + [O, nb, 16])
            inv[name + ".dm"] = ("F16", lead + [O, nb, 1])
        elif kind in (A8, A4):
            bits, group = (8, 64) if kind == A8 else (4, 32)
            inv[name + ".weight"] = ("U32", lead + [O, K * bits // 32])
            inv[name + ".scales"] = ("BF16", lead + [O, K // group])
            inv[name + ".biases"] = ("BF16", lead + [O, K // group])
        else:
            inv[name + ".weight"] = ("BF16", lead + [O, K])

    pub = mix == "published"
    P = "language_model.model."
    mod(P + "embed_tokens", A8, V, H)
    mod("language_model.lm_head", Q4K if pub else A8, V, H)
    inv[P + "norm.weight"] = ("BF16", [H])
    for i in range(cfg.n_layers):
        lp = P + "layers.%d." % i
        inv[lp + "input_layernorm.weight"] = ("BF16", [H])
        inv[lp + "post_attention_layernorm.weight"] = ("BF16", [H])
        if (i + 1) % cfg.full_attn_interval != 0:
            a = lp + "linear_attn."
            lin = Q4K if pub else A8
            mod(a + "in_proj_qkv", lin, D, H)
            mod(a + "in_proj_z", lin, VD, H)
            mod(a + "out_proj", lin, H, VD)
            mod(a + "in_proj_a", BF16, cfg.gdn_v_heads, H)
            mod(a + "in_proj_b", BF16, cfg.gdn_v_heads, H)
            inv[a + "conv1d.weight"] = ("BF16", [D, cfg.gdn_conv_kernel, 1])
            inv[a + "dt_bias"] = ("BF16", [cfg.gdn_v_heads])
            inv[a + "A_log"] = ("BF16", [cfg.gdn_v_heads])
            inv[a + "norm.weight"] = ("BF16", [cfg.gdn_head_dim])
        else:
            a = lp + "self_attn."
            att = Q6K if pub else A8
            mod(a + "q_proj", att, 2 * QD, H)
            mod(a + "k_proj", att, KVD, H)
            mod(a + "v_proj", att, KVD, H)
            mod(a + "o_proj", att, H, QD)
            inv[a + "q_norm.weight"] = ("BF16", [cfg.head_dim])
            inv[a + "k_norm.weight"] = ("BF16", [cfg.head_dim])
        m = lp + "mlp."
        late = i >= 32   # the artifact's 8-bit side: layers 32..39
        if pub:
            router, gu, dn, sgu, sdn = Q6K, (Q6K if late else Q4K), (Q6K if late else Q4K), (Q6K if late else A4), (Q6K if late else A4)
        else:
            router, gu, dn, sgu, sdn = A8, Q4K, Q6K, Q4K, Q6K
        mod(m + "gate", router, E, H)
        mod(m + "switch_mlp.gate_proj", gu, I, H, (E,))
        mod(m + "switch_mlp.up_proj", gu, I, H, (E,))
        mod(m + "switch_mlp.down_proj", dn, H, I, (E,))
        mod(m + "shared_expert.gate_proj", sgu, SI, H)
        mod(m + "shared_expert.up_proj", sgu, SI, H)
        mod(m + "shared_expert.down_proj", sdn, H, SI)
        mod(m + "shared_expert_gate", A8, 1, H)
    return inv
