"""TEST INFRASTRUCTURE: ctypes binding of the CPU oracle (liborn_oracle.so).

Used by the tests, by the smoke check and by the CPU-baseline leg of the
benchmark.  Nothing under the package imports this.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ORACLE_DIR = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(ORACLE_DIR, "liborn_oracle.so")

Q4K, Q6K, A8, BF16, A4 = 0, 1, 2, 3, 4


class Lin(C.Structure):
    _fields_ = [("kind", C.c_int32), ("E", C.c_int32), ("O", C.c_int32), ("K", C.c_int32),
                ("w", C.c_void_p), ("s", C.c_void_p), ("b", C.c_void_p)]


class Config(C.Structure):
    _fields_ = [
        ("hidden", C.c_int32), ("n_layers", C.c_int32), ("full_attn_interval", C.c_int32),
        ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("rope_dims", C.c_int32), ("rope_theta", C.c_float),
        ("gdn_k_heads", C.c_int32), ("gdn_v_heads", C.c_int32), ("gdn_head_dim", C.c_int32),
        ("gdn_conv_kernel", C.c_int32),
        ("n_experts", C.c_int32), ("top_k", C.c_int32), ("expert_inter", C.c_int32),
        ("shared_inter", C.c_int32), ("norm_topk_prob", C.c_int32),
        ("vocab", C.c_int32), ("rms_eps", C.c_float), ("max_ctx", C.c_int32),
    ]


class Moe(C.Structure):
    _fields_ = [(n, Lin) for n in ("gate", "sw_gate", "sw_up", "sw_down", "sh_gate", "sh_up", "sh_down", "sh_egate")]


class MtpStats(C.Structure):
    _fields_ = [("cycles", C.c_int32), ("drafted", C.c_int32), ("accepted", C.c_int32),
                ("reached_by_depth", C.c_int32 * 8), ("accepted_by_depth", C.c_int32 * 8)]


class Force(C.Structure):
    _fields_ = [("stream", C.c_void_p), ("len", C.c_int32), ("p", C.c_float), ("seed", C.c_uint64)]


def build():
    srcs = [os.path.join(ORACLE_DIR, f) for f in os.listdir(ORACLE_DIR) if f.endswith((".c", ".h"))]
    if (not os.path.exists(LIB)) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in srcs):
        subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(LIB)
        _lib.orc_row_dot.restype = C.c_float
        _lib.orc_logsumexp.restype = C.c_uint16
        _lib.orc_greedy_token.restype = C.c_uint32
        _lib.orc_sumsq.restype = C.c_float
        _lib.orc_model_new.restype = C.c_void_p
        _lib.orc_cache_new.restype = C.c_void_p
        _lib.orc_model_new.argtypes = [C.POINTER(Config)]
        _lib.orc_model_free.argtypes = [C.c_void_p]
        _lib.orc_cache_new.argtypes = [C.c_void_p]
        _lib.orc_cache_free.argtypes = [C.c_void_p]
        _lib.orc_cache_offset.argtypes = [C.c_void_p]
        _lib.orc_model_set.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                       C.c_void_p, C.c_void_p, C.c_void_p]
        _lib.orc_model_set_frspec.argtypes = [C.c_void_p, C.POINTER(Lin), C.c_void_p, C.c_int]
        _lib.orc_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        _lib.orc_head_greedy.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        _lib.orc_generate.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        _lib.orc_generate_mtp.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_int, C.POINTER(Force), C.c_void_p,
                                          C.POINTER(MtpStats)]
    return _lib


def ptr(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


class Weights:
    """A weight matrix in artifact layout held as numpy arrays (kept alive here)."""

    def __init__(self, kind, E, O, K, w, s=None, b=None):
        self.kind, self.E, self.O, self.K = kind, E, O, K
        self.w = np.ascontiguousarray(w)
        self.s = None if s is None else np.ascontiguousarray(s)
        self.b = None if b is None else np.ascontiguousarray(b)

    def lin(self):
        return Lin(self.kind, self.E, self.O, self.K, self.w.ctypes.data,
                   0 if self.s is None else self.s.ctypes.data, 0 if self.b is None else self.b.ctypes.data)


def gemv(W, x_bf, M, f32=False):
    L = W.lin()
    x_bf = np.ascontiguousarray(x_bf, np.uint16)
    yf = np.zeros((M, W.O), np.float32) if f32 else None
    yb = np.zeros((M, W.O), np.uint16)
    lib().orc_gemv(C.byref(L), ptr(x_bf), M, ptr(yf), ptr(yb))
    return yf if f32 else yb


def gather_gemv(W, x_bf, lhs, rhs):
    L = W.lin()
    rows = len(lhs)
    y = np.zeros((rows, W.O), np.uint16)
    x_bf = np.ascontiguousarray(x_bf, np.uint16)
    lhs = np.ascontiguousarray(lhs, np.uint32)
    rhs = np.ascontiguousarray(rhs, np.uint32)
    lib().orc_gather_gemv(C.byref(L), ptr(x_bf), ptr(lhs), ptr(rhs), rows, ptr(y))
    return y


def q4k_dequantize(qs, scales, dm):
    n = scales.size // 12
    out = np.zeros((n, 256), np.float32)
    lib().orc_q4k_dequantize(ptr(qs), ptr(scales), ptr(dm), C.c_int64(n), ptr(out))
    return out


def q4k_fields(qs, scales):
    n = scales.size // 12
    sc = np.zeros((n, 8), np.uint8)
    mn = np.zeros((n, 8), np.uint8)
    q = np.zeros((n, 256), np.uint8)
    lib().orc_q4k_fields(ptr(qs), ptr(scales), C.c_int64(n), ptr(sc), ptr(mn), ptr(q))
    return sc, mn, q


def q6k_dequantize(w, scales, dm):
    n = scales.size // 16
    out = np.zeros((n, 256), np.float32)
    lib().orc_q6k_dequantize(ptr(w), ptr(scales), ptr(dm), C.c_int64(n), ptr(out))
    return out


def embedding(W, ids):
    L = W.lin()
    ids = np.ascontiguousarray(ids, np.uint32)
    out = np.zeros((len(ids), W.K), np.uint16)
    lib().orc_embedding_a8(C.byref(L), ptr(ids), len(ids), ptr(out))
    return out


def rms_norm(x, w, rows, n, eps):
    out = np.zeros((rows, n), np.uint16)
    lib().orc_rms_norm(ptr(x), ptr(w), rows, n, C.c_float(eps), ptr(out))
    return out


def add_rms_norm(a, b, w, rows, n, eps):
    h = np.zeros((rows, n), np.uint16)
    out = np.zeros((rows, n), np.uint16)
    lib().orc_add_rms_norm(ptr(a), ptr(b), ptr(w), rows, n, C.c_float(eps), ptr(h), ptr(out))
    return h, out


def rms_norm_gated(x, w, z, rows, n, eps):
    out = np.zeros((rows, n), np.uint16)
    lib().orc_rms_norm_gated(ptr(x), ptr(w), ptr(z), rows, n, C.c_float(eps), ptr(out))
    return out


def sigmoid_gate(gate, x, n, inner):
    out = np.zeros(n, np.uint16)
    lib().orc_sigmoid_gate(ptr(gate), ptr(x), n, inner, ptr(out))
    return out


def swiglu(g, u):
    out = np.zeros(g.size, np.uint16)
    lib().orc_swiglu(ptr(g), ptr(u), g.size, ptr(out))
    return out


def softmax_precise(x, rows, n):
    out = np.zeros((rows, n), np.uint16)
    lib().orc_softmax_precise(ptr(x), rows, n, ptr(out))
    return out


def router_topk(gates, rows, n, k):
    inds = np.zeros((rows, k), np.uint32)
    scores = np.zeros((rows, k), np.uint16)
    lib().orc_router_topk(ptr(gates), rows, n, k, ptr(inds), ptr(scores))
    return inds, scores


def moe_combine(scores, y, gate, shared, T, k, dim, normalize):
    out = np.zeros((T, dim), np.uint16)
    lib().orc_moe_combine(ptr(scores), ptr(y), ptr(gate), ptr(shared), T, k, dim, normalize, ptr(out))
    return out


def moe_block(ws, x, T, top_k, norm_topk):
    """ws: dict of the eight Weights keyed like the Moe struct fields."""
    m = Moe(**{k: ws[k].lin() for k in ("gate", "sw_gate", "sw_up", "sw_down", "sh_gate", "sh_up", "sh_down", "sh_egate")})
    H = ws["gate"].K
    out = np.zeros((T, H), np.uint16)
    inds = np.zeros((T, top_k), np.uint32)
    lib().orc_moe_block(C.byref(m), ptr(x), T, top_k, norm_topk, ptr(out), ptr(inds))
    return out, inds


def gdn_front(conv_state, qkv, cw, a, b, a_log, dt_bias, T, Hk, Hv, Dh, Kc, eps=1e-6):
    D = 2 * Hk * Dh + Hv * Dh
    conv_next = np.zeros((Kc - 1, D), np.uint16)
    q = np.zeros((T, Hk, Dh), np.uint16)
    k = np.zeros((T, Hk, Dh), np.uint16)
    v = np.zeros((T, Hv, Dh), np.uint16)
    beta = np.zeros((T, Hv), np.uint16)
    g = np.zeros((T, Hv), np.float32)
    lib().orc_gdn_front(ptr(conv_state), ptr(qkv), ptr(cw), ptr(a), ptr(b), ptr(a_log), ptr(dt_bias), T, Hk,
                        Hv, Dh, Kc, C.c_float(eps), ptr(conv_next), ptr(q), ptr(k), ptr(v), ptr(beta), ptr(g))
    return conv_next, q, k, v, beta, g


def gated_delta(q, k, v, g, beta, state, T, Hk, Hv, want_snaps=False):
    """state is updated in place (float32 [Hv,128,128])."""
    y = np.zeros((T, Hv, 128), np.uint16)
    snaps = np.zeros((T,) + state.shape, np.float32) if want_snaps else None
    lib().orc_gated_delta(ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(state), T, Hk, Hv, ptr(y), ptr(snaps))
    return (y, snaps) if want_snaps else y


def rope(x, T, H, hd, dims, theta, offset):
    x = np.ascontiguousarray(x, np.uint16).copy()
    lnb = np.float32(np.log(np.float64(np.float32(theta))) / (dims // 2))
    lib().orc_rope(ptr(x), T, H, hd, dims, C.c_float(lnb), offset)
    return x


def sdpa_decode(q, kc, vc, T, Hq, Hkv, hd, cap, offset, scale):
    out = np.zeros((T, Hq, hd), np.uint16)
    lib().orc_sdpa_decode(ptr(q), ptr(kc), ptr(vc), T, Hq, Hkv, hd, cap, offset, C.c_float(scale), ptr(out))
    return out


def greedy_token(logits, normalize):
    logits = np.ascontiguousarray(logits, np.uint16)
    return int(lib().orc_greedy_token(ptr(logits), logits.size, int(normalize)))


def logsumexp(logits):
    logits = np.ascontiguousarray(logits, np.uint16)
    return int(lib().orc_logsumexp(ptr(logits), logits.size))


class Model:
    """orc_model over a dict name -> Weights | numpy uint16 tensor."""

    def __init__(self, cfg, weights):
        self.cfg = Config(**{f[0]: getattr(cfg, f[0]) for f in Config._fields_})
        self.weights = weights  # keeps the numpy arrays alive
        self.h = C.c_void_p(lib().orc_model_new(C.byref(self.cfg)))
        for name, w in weights.items():
            if isinstance(w, Weights):
                rc = lib().orc_model_set(self.h, name.encode(), w.kind, w.E, w.O, w.K, ptr(w.w), ptr(w.s), ptr(w.b))
            else:
                rc = lib().orc_model_set(self.h, name.encode(), BF16, 1, 1, w.size, ptr(w), None, None)
            assert rc == 0, "oracle does not know the tensor %r" % name
        self._fr = None

    def set_frspec(self, pruned, ids):
        ids = np.ascontiguousarray(ids, np.uint32)
        L = pruned.lin()
        self._fr = (pruned, ids, L)
        lib().orc_model_set_frspec(self.h, C.byref(L), ptr(ids), len(ids))

    def new_cache(self):
        return C.c_void_p(lib().orc_cache_new(self.h))

    def free_cache(self, c):
        lib().orc_cache_free(c)

    def forward(self, cache, ids):
        ids = np.ascontiguousarray(ids, np.uint32)
        if lib().orc_cache_offset(cache) + len(ids) > self.cfg.max_ctx:
            raise ValueError("oracle forward: the window would pass max_ctx=%d" % self.cfg.max_ctx)
        out = np.zeros((len(ids), self.cfg.hidden), np.uint16)
        lib().orc_forward(self.h, cache, ptr(ids), len(ids), ptr(out), None)
        return out

    def head_greedy(self, hidden, T, want_logits=False):
        toks = np.zeros(T, np.uint32)
        logits = np.zeros((T, self.cfg.vocab), np.uint16) if want_logits else None
        hidden = np.ascontiguousarray(hidden, np.uint16)
        lib().orc_head_greedy(self.h, ptr(hidden), T, ptr(toks), ptr(logits))
        return (toks, logits) if want_logits else toks

    def generate(self, prompt, max_tokens):
        cache = self.new_cache()
        prompt = np.ascontiguousarray(prompt, np.uint32)
        out = np.zeros(max_tokens, np.uint32)
        n = lib().orc_generate(self.h, cache, ptr(prompt), len(prompt), max_tokens, ptr(out))
        self.free_cache(cache)
        return out[:n].tolist()

    def generate_mtp(self, prompt, depth, max_tokens, policy=1, frspec=False, force=None):
        cache = self.new_cache()
        prompt = np.ascontiguousarray(prompt, np.uint32)
        out = np.zeros(max_tokens + 8, np.uint32)
        stats = MtpStats()
        fd = None
        if force is not None:
            stream, p, seed = force
            stream = np.ascontiguousarray(stream, np.uint32)
            fd = Force(stream.ctypes.data, len(stream), p, seed)
        n = lib().orc_generate_mtp(self.h, cache, ptr(prompt), len(prompt), depth, max_tokens, policy,
                                   int(bool(frspec)), C.byref(fd) if fd is not None else None, ptr(out),
                                   C.byref(stats))
        self.free_cache(cache)
        return out[:n].tolist(), stats

    def free(self):
        if self.h:
            lib().orc_model_free(self.h)
            self.h = None


def model_weight_names(cfg):
    """(linears, tensors): every weight name of a model with this config."""
    lin, ten = ["embed_tokens", "lm_head"], ["norm.weight"]
    moe = ["gate", "switch_mlp.gate_proj", "switch_mlp.up_proj", "switch_mlp.down_proj",
           "shared_expert.gate_proj", "shared_expert.up_proj", "shared_expert.down_proj", "shared_expert_gate"]
    for i in range(cfg.n_layers):
        lp = "layers.%d." % i
        ten += [lp + "input_layernorm.weight", lp + "post_attention_layernorm.weight"]
        if (i + 1) % cfg.full_attn_interval != 0:
            a = lp + "linear_attn."
            lin += [a + n for n in ("in_proj_qkv", "in_proj_z", "in_proj_a.weight", "in_proj_b.weight", "out_proj")]
            ten += [a + n for n in ("conv1d.weight", "dt_bias", "A_log", "norm.weight")]
        else:
            a = lp + "self_attn."
            lin += [a + n for n in ("q_proj", "k_proj", "v_proj", "o_proj")]
            ten += [a + "q_norm.weight", a + "k_norm.weight"]
        lin += [lp + "mlp." + n for n in moe]
    lp = "mtp.layers.0."
    ten += ["mtp.pre_fc_norm_embedding.weight", "mtp.pre_fc_norm_hidden.weight", "mtp.norm.weight",
            lp + "input_layernorm.weight", lp + "post_attention_layernorm.weight",
            lp + "self_attn.q_norm.weight", lp + "self_attn.k_norm.weight"]
    lin += ["mtp.fc.weight"] + [lp + "self_attn.%s_proj.weight" % c for c in "qkvo"] + [lp + "mlp." + n for n in moe]
    return lin, ten


def export_gpu_model(gpu_model):
    """Download every weight of a CUDA-side model into an oracle Model (the same
    bytes on both sides)."""
    cfg = gpu_model.cfg
    lins, tens = model_weight_names(cfg)
    W = {}
    for n in lins:
        L = gpu_model.get_linear(n)
        w, s, b = L.export()
        W[n] = Weights(L.kind, L.E, L.O, L.K, w, s if s.size else None, b if b.size else None)
    for n in tens:
        W[n] = gpu_model.get_tensor(n)
    return Model(cfg, W)
