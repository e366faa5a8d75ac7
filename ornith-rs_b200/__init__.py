"""Host-side mirror of ornith-rs's decode API over the sm_100a CUDA library.

The reference crate is Rust; its toolchain is not available where this was
built, so the code above the C ABI that a Rust caller would own (model, caches,
generation loops) is C++ inside libornith_cuda.so, and this module is the thin
ctypes harness tests and benchmarks drive it through.  Names follow the
reference: `Linear` (src/ops/linear.rs), `TextModel` / `make_cache`
(src/model/qwen3_5.rs), `generate_step` (src/generate.rs), `generate_step_mtp`
and `MtpStats` (src/mtp_generate.rs), `FrSpec` (src/frspec.rs).

Activations are bfloat16 carried as numpy uint16; device buffers are `DevBuf`.
There is no CPU fallback: every call runs a CUDA kernel or raises.
"""
import ctypes as C

import numpy as np

from . import _ffi
from ._ffi import A4, A8, BF16, POLICY_COMMITTED, POLICY_CYCLE, Q4K, Q6K, Config, ForceDraft, MtpStats, Prof

__all__ = [
    "Context", "DevBuf", "Linear", "TextModel", "Cache", "Config", "MtpStats", "OrnError",
    "Q4K", "Q6K", "A8", "BF16", "A4", "POLICY_CYCLE", "POLICY_COMMITTED", "generate_step",
    "generate_step_mtp", "qwen35_config", "lib",
]


class OrnError(RuntimeError):
    pass


def lib():
    return _ffi.load()


def qwen35_config(max_ctx=512, **over):
    """Qwen3.5-MoE 35B-A3B text dimensions (reference: baseline/config.json,
    src/model/config.rs:171-184)."""
    c = Config(hidden=2048, n_layers=40, full_attn_interval=4, n_heads=16, n_kv_heads=2, head_dim=256,
               rope_dims=64, rope_theta=1e7, gdn_k_heads=16, gdn_v_heads=32, gdn_head_dim=128,
               gdn_conv_kernel=4, n_experts=256, top_k=8, expert_inter=512, shared_inter=512,
               norm_topk_prob=1, vocab=248320, rms_eps=1e-6, max_ctx=max_ctx)
    for k, v in over.items():
        setattr(c, k, v)
    return c


class Context:
    """orn_ctx: one device, one stream (the reference's metal::Context)."""

    def __init__(self, device=0):
        self.device = device
        self._lib = lib()
        h = C.c_void_p()
        rc = self._lib.orn_ctx_create(device, C.byref(h))
        if rc != 0:
            raise OrnError("orn_ctx_create(%d) failed with status %d (is a CUDA device present?)" % (device, rc))
        self.h = h

    def check(self, rc, what=""):
        if rc != 0:
            msg = self._lib.orn_last_error(self.h)
            raise OrnError("%s: status %d: %s" % (what, rc, msg.decode() if msg else ""))

    def sync(self):
        self.check(self._lib.orn_sync(self.h), "orn_sync")

    def alloc(self, nbytes):
        p = C.c_void_p()
        self.check(self._lib.orn_alloc(self.h, nbytes, C.byref(p)), "orn_alloc")
        return DevBuf(self, p, nbytes)

    def empty(self, shape, dtype):
        dtype = np.dtype(dtype)
        n = int(np.prod(shape)) * dtype.itemsize
        b = self.alloc(n)
        b.shape, b.dtype = tuple(shape), dtype
        return b

    def zeros(self, shape, dtype):
        b = self.empty(shape, dtype)
        self.check(self._lib.orn_memset(self.h, b.ptr, 0, b.nbytes), "orn_memset")
        return b

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        b = self.alloc(arr.nbytes)
        b.shape, b.dtype = arr.shape, arr.dtype
        if arr.nbytes:
            self.check(self._lib.orn_upload(self.h, b.ptr, arr.ctypes.data, arr.nbytes), "orn_upload")
        return b

    def launches(self):
        n = C.c_int64()
        self.check(self._lib.orn_ctx_launches(self.h, C.byref(n)), "orn_ctx_launches")
        return n.value

    def timer_start(self):
        self.check(self._lib.orn_timer_start(self.h), "orn_timer_start")

    def timer_stop(self):
        ms = C.c_float()
        self.check(self._lib.orn_timer_stop(self.h, C.byref(ms)), "orn_timer_stop")
        return ms.value

    def ktime_begin(self):
        """Per-kernel device times from here on (eager launches, an event after each)."""
        self.check(self._lib.orn_ctx_ktime_begin(self.h), "orn_ctx_ktime_begin")

    def ktime_end(self):
        """-> {label: (launches, total_ms)} since ktime_begin."""
        buf = C.create_string_buffer(1 << 16)
        self.check(self._lib.orn_ctx_ktime_end(self.h, buf, len(buf)), "orn_ctx_ktime_end")
        out = {}
        for line in buf.value.decode().splitlines():
            name, n, ms = line.split("\t")
            out[name] = (int(n), float(ms))
        return out

    def close(self):
        if self.h:
            self._lib.orn_ctx_destroy(self.h)
            self.h = None


class DevBuf:
    """A device allocation with a numpy-style shape and dtype."""

    def __init__(self, ctx, ptr, nbytes):
        self.ctx, self.ptr, self.nbytes = ctx, ptr, nbytes
        self.shape, self.dtype = (nbytes,), np.dtype(np.uint8)

    def numpy(self):
        out = np.empty(self.shape, self.dtype)
        if out.nbytes:
            self.ctx.check(self.ctx._lib.orn_download(self.ctx.h, out.ctypes.data, self.ptr, out.nbytes),
                           "orn_download")
        return out

    def set(self, arr):
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes <= self.nbytes
        self.ctx.check(self.ctx._lib.orn_upload(self.ctx.h, self.ptr, arr.ctypes.data, arr.nbytes), "orn_upload")

    def at(self, byte_offset):
        return C.c_void_p(self.ptr.value + byte_offset)

    def free(self):
        if self.ptr:
            self.ctx._lib.orn_free(self.ctx.h, self.ptr)
            self.ptr = None


def _p(x):
    if x is None:
        return None
    if isinstance(x, DevBuf):
        return x.ptr
    return x


class Linear:
    """A weight matrix [E, O, K] resident in HBM (KMatrix / QuantMatrix / dense
    Array of the reference)."""

    def __init__(self, ctx, handle, kind, E, O, K, owned=True):
        self.ctx, self.h, self.kind, self.E, self.O, self.K, self.owned = ctx, handle, kind, E, O, K, owned

    @classmethod
    def from_numpy(cls, ctx, kind, w, s=None, b=None, E=1, O=None, K=None):
        w = np.ascontiguousarray(w)
        s = None if s is None else np.ascontiguousarray(s)
        b = None if b is None else np.ascontiguousarray(b)
        h = C.c_void_p()
        rc = ctx._lib.orn_linear_create(ctx.h, kind, E, O, K, w.ctypes.data,
                                        None if s is None else s.ctypes.data,
                                        None if b is None else b.ctypes.data, C.byref(h))
        ctx.check(rc, "orn_linear_create")
        return cls(ctx, h, kind, E, O, K)

    @classmethod
    def random(cls, ctx, kind, E, O, K, seed, std=0.02):
        h = C.c_void_p()
        ctx.check(ctx._lib.orn_linear_create_random(ctx.h, kind, E, O, K, seed, std, C.byref(h)),
                  "orn_linear_create_random")
        return cls(ctx, h, kind, E, O, K)

    def export(self):
        """Artifact-layout tensors (w, s, b) as numpy uint8 arrays."""
        a, bb, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
        self.ctx._lib.orn_linear_sizes(self.h, C.byref(a), C.byref(bb), C.byref(c))
        w = np.empty(a.value, np.uint8)
        s = np.empty(bb.value, np.uint8)
        b = np.empty(c.value, np.uint8)
        self.ctx.check(self.ctx._lib.orn_linear_export(self.ctx.h, self.h, w.ctypes.data,
                                                       s.ctypes.data if s.size else None,
                                                       b.ctypes.data if b.size else None),
                       "orn_linear_export")
        return w, s, b

    def gather_rows(self, ids):
        ids = np.ascontiguousarray(ids, np.uint32)
        h = C.c_void_p()
        self.ctx.check(self.ctx._lib.orn_linear_gather_rows(self.ctx.h, self.h, ids.ctypes.data, len(ids),
                                                            C.byref(h)), "orn_linear_gather_rows")
        return Linear(self.ctx, h, self.kind, 1, len(ids), self.K)

    def matmul(self, x, M, out_f32=False):
        """Linear::matmul for M <= 4 rows (src/ops/linear.rs:23-80)."""
        y = self.ctx.empty((M, self.O), np.float32 if out_f32 else np.uint16)
        self.ctx.check(self.ctx._lib.orn_gemv(self.ctx.h, self.h, _p(x), M, y.ptr, int(out_f32)), "orn_gemv")
        return y

    def matmul_wide(self, x, M, out_f32=False):
        """Linear::matmul at prompt width (tensor cores; agrees with matmul to rounding)."""
        y = self.ctx.empty((M, self.O), np.float32 if out_f32 else np.uint16)
        self.ctx.check(self.ctx._lib.orn_gemm(self.ctx.h, self.h, _p(x), M, y.ptr, int(out_f32)), "orn_gemm")
        return y

    def gather_matmul_wide(self, x, lhs, rhs, rows, out_f32=False):
        y = self.ctx.empty((rows, self.O), np.float32 if out_f32 else np.uint16)
        self.ctx.check(self.ctx._lib.orn_gather_gemm(self.ctx.h, self.h, _p(x), _p(lhs), _p(rhs), rows, y.ptr,
                                                     int(out_f32)), "orn_gather_gemm")
        return y

    def gather_matmul(self, x, lhs, rhs, rows):
        y = self.ctx.empty((rows, self.O), np.uint16)
        self.ctx.check(self.ctx._lib.orn_gather_gemv(self.ctx.h, self.h, _p(x), _p(lhs), _p(rhs), rows, y.ptr),
                       "orn_gather_gemv")
        return y

    def dequantize(self, e=0):
        out = self.ctx.empty((self.O, self.K), np.float32)
        self.ctx.check(self.ctx._lib.orn_kq_dequantize(self.ctx.h, self.h, e, out.ptr), "orn_kq_dequantize")
        return out

    def free(self):
        if self.h and self.owned:
            self.ctx._lib.orn_linear_destroy(self.ctx.h, self.h)
        self.h = None


class TextModel:
    """orn_model: the trunk plus the MTP head (TextModel + MtpHead of the reference)."""

    def __init__(self, ctx, cfg):
        self.ctx, self.cfg = ctx, cfg
        h = C.c_void_p()
        ctx.check(ctx._lib.orn_model_create(ctx.h, C.byref(cfg), C.byref(h)), "orn_model_create")
        self.h = h

    @classmethod
    def load(cls, ctx, directory, max_ctx=512):
        """TextModel::load + MtpHead::load from safetensors shards (src/weights.rs:41-279)."""
        h = C.c_void_p()
        ctx.check(ctx._lib.orn_model_load(ctx.h, directory.encode(), max_ctx, C.byref(h)), "orn_model_load")
        self = cls.__new__(cls)
        self.ctx, self.h = ctx, h
        self.cfg = Config()
        ctx.check(ctx._lib.orn_model_config(h, C.byref(self.cfg)), "orn_model_config")
        return self

    def init_random(self, seed):
        self.ctx.check(self.ctx._lib.orn_model_init_random(self.h, seed), "orn_model_init_random")

    def set_linear(self, name, lin):
        self.ctx.check(self.ctx._lib.orn_model_set_linear(self.h, name.encode(), lin.h), "orn_model_set_linear")
        lin.owned = False

    def set_tensor(self, name, arr):
        arr = np.ascontiguousarray(arr, np.uint16)
        self.ctx.check(self.ctx._lib.orn_model_set_tensor(self.h, name.encode(), arr.ctypes.data, arr.size),
                       "orn_model_set_tensor")

    def get_linear(self, name):
        h = C.c_void_p()
        self.ctx.check(self.ctx._lib.orn_model_get_linear(self.h, name.encode(), C.byref(h)), "orn_model_get_linear")
        k, e, o, kk = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
        self.ctx._lib.orn_linear_info(h, C.byref(k), C.byref(e), C.byref(o), C.byref(kk))
        return Linear(self.ctx, h, k.value, e.value, o.value, kk.value, owned=False)

    def get_tensor(self, name):
        p, n = C.c_void_p(), C.c_size_t()
        self.ctx.check(self.ctx._lib.orn_model_get_tensor(self.h, name.encode(), C.byref(p), C.byref(n)),
                       "orn_model_get_tensor")
        b = DevBuf(self.ctx, p, n.value * 2)
        b.shape, b.dtype = (n.value,), np.dtype(np.uint16)
        return b.numpy()

    def weight_bytes(self):
        return self.ctx._lib.orn_model_weight_bytes(self.h)

    def set_frspec(self, ids):
        ids = np.ascontiguousarray(ids, np.uint32)
        self.ctx.check(self.ctx._lib.orn_frspec_set(self.h, ids.ctypes.data, len(ids)), "orn_frspec_set")

    def load_frspec(self, path):
        self.ctx.check(self.ctx._lib.orn_frspec_load(self.h, path.encode()), "orn_frspec_load")

    def make_cache(self):
        return Cache(self)

    def forward(self, cache, ids, capture=False):
        """forward_hidden / forward_capture: returns the post-norm hidden rows (device)."""
        ids = np.ascontiguousarray(ids, np.uint32)
        T = len(ids)
        out = self.ctx.empty((T, self.cfg.hidden), np.uint16)
        if capture:
            rc = self.ctx._lib.orn_forward_capture(self.h, cache.h, ids.ctypes.data, T, out.ptr)
        else:
            rc = self.ctx._lib.orn_forward(self.h, cache.h, ids.ctypes.data, T, out.ptr, None)
        self.ctx.check(rc, "orn_forward")
        return out

    def prefill(self, cache, ids, prefill_step=2048, want_hidden=False):
        """generate::prefill over all ids; chunks of 64 rows or more run on the tensor cores.
        want_hidden: returns the post-norm hidden rows [n, hidden] (device)."""
        ids = np.ascontiguousarray(ids, np.uint32)
        out = self.ctx.empty((len(ids), self.cfg.hidden), np.uint16) if want_hidden else None
        self.ctx.check(self.ctx._lib.orn_prefill(self.h, cache.h, ids.ctypes.data, len(ids), prefill_step, _p(out)),
                       "orn_prefill")
        return out

    def mtp_forward(self, cache, hidden, ids, kv_only=False):
        """MtpHead::forward for len(ids) rows; returns the draft (raw-logit argmax of the last row) or None."""
        ids = np.ascontiguousarray(ids, np.uint32)
        out = np.zeros(1, np.uint32)
        self.ctx.check(self.ctx._lib.orn_mtp_forward(self.h, cache.h, _p(hidden), ids.ctypes.data, len(ids), int(bool(kv_only)),
                                                     None if kv_only else out.ctypes.data), "orn_mtp_forward")
        return None if kv_only else int(out[0])

    def head_greedy(self, hidden, T, want_logits=False):
        toks = np.zeros(T, np.uint32)
        logits = self.ctx.empty((T, self.cfg.vocab), np.uint16) if want_logits else None
        self.ctx.check(self.ctx._lib.orn_head_greedy(self.h, _p(hidden), T, toks.ctypes.data, _p(logits)),
                       "orn_head_greedy")
        return (toks, logits) if want_logits else toks

    def prof(self):
        p = Prof()
        self.ctx.check(self.ctx._lib.orn_get_prof(self.h, C.byref(p)), "orn_get_prof")
        return p

    def free(self):
        if self.h:
            self.ctx._lib.orn_model_destroy(self.h)
            self.h = None


class Batch:
    """orn_batch: B concurrent sequences stepping verify windows of up to t_max rows through the
    whole trunk in one pass over the weights (csrc/batch.cu).  `ep` is an `ep.LibEp` group (None:
    this GPU alone); with several ranks every rank holds its own B sequences and serves its share
    of every layer's experts, and forward() is collective.  exact=True keeps every product on the
    row-invariant mat-vec (bit-identical to the single-sequence engine)."""

    def __init__(self, model, B, t_max=2, cap=256, exact=False, split_attn=False):
        self.model, self.ctx, self.B, self.t_max, self.cap = model, model.ctx, B, t_max, cap
        h = C.c_void_p()
        self.ctx.check(self.ctx._lib.orn_batch_create(model.h, B, t_max, cap, (1 if exact else 0) | (2 if split_attn else 0),
                                                      C.byref(h)),
                       "orn_batch_create")
        self.h = h

    def reset(self):
        self.ctx.check(self.ctx._lib.orn_batch_reset(self.h), "orn_batch_reset")

    def fill_random(self, ctx_len, seed=1):
        self.ctx.check(self.ctx._lib.orn_batch_fill_random(self.h, ctx_len, seed), "orn_batch_fill_random")

    def positions(self):
        out = np.zeros(self.B, np.int32)
        self.ctx.check(self.ctx._lib.orn_batch_positions(self.h, out.ctypes.data), "orn_batch_positions")
        return out

    def forward(self, ids, ep=None, want_hidden=False, want_targets=True):
        """ids [B, T] -> (greedy targets [B, T] or None, post-norm hidden rows [B*T, hidden] on the device or None)."""
        ids = np.ascontiguousarray(ids, np.uint32)
        if ids.ndim != 2 or ids.shape[0] != self.B:
            raise ValueError("Batch.forward: ids must be [B, T]")
        T = ids.shape[1]
        hid = self.ctx.empty((self.B * T, self.model.cfg.hidden), np.uint16) if want_hidden else None
        tg = np.zeros((self.B, T), np.uint32) if want_targets else None
        self.ctx.check(self.ctx._lib.orn_batch_forward(self.h, None if ep is None else ep.h, ids.ctypes.data, T, _p(hid),
                                                       None if tg is None else tg.ctypes.data), "orn_batch_forward")
        return tg, hid

    def mtp_draft(self, primary, ep=None):
        """One draft token per sequence from the MTP head (depth 1): primary [B] -> drafts [B]."""
        primary = np.ascontiguousarray(primary, np.uint32)
        if primary.shape != (self.B,):
            raise ValueError("Batch.mtp_draft: one primary token per sequence")
        out = np.zeros(self.B, np.uint32)
        self.ctx.check(self.ctx._lib.orn_batch_mtp_draft(self.h, None if ep is None else ep.h, primary.ctypes.data,
                                                         out.ctypes.data), "orn_batch_mtp_draft")
        return out

    def commit(self, keep):
        keep = np.ascontiguousarray(keep, np.int32)
        if keep.shape != (self.B,):
            raise ValueError("Batch.commit: one keep per sequence")
        self.ctx.check(self.ctx._lib.orn_batch_commit(self.h, keep.ctypes.data), "orn_batch_commit")

    def free(self):
        if self.h:
            self.ctx._lib.orn_batch_destroy(self.h)
            self.h = None


class Cache:
    """orn_cache: KvCache + GdnCache per layer and the MTP head's KvCache (src/model/cache.rs)."""

    def __init__(self, model):
        self.model = model
        h = C.c_void_p()
        model.ctx.check(model.ctx._lib.orn_cache_create(model.h, C.byref(h)), "orn_cache_create")
        self.h = h

    def reset(self):
        self.model.ctx.check(self.model.ctx._lib.orn_cache_reset(self.h), "orn_cache_reset")

    def rewind(self, keep):
        self.model.ctx.check(self.model.ctx._lib.orn_cache_rewind(self.h, keep), "orn_cache_rewind")

    @property
    def offset(self):
        return self.model.ctx._lib.orn_cache_offset(self.h)

    def free(self):
        if self.h:
            self.model.ctx._lib.orn_cache_destroy(self.h)
            self.h = None


def add_norm_gemv(ctx, a, b, w, M, K, eps, lins, want_h=False, want_normed=False):
    """add_rms_norm followed by up to four Linear::matmul over the same rows, one
    persistent kernel (src/model/qwen3_5.rs:478-565, norm.rs:19-220, linear.rs:23-80).
    Returns (outs, h, normed)."""
    n = len(lins)
    outs = [ctx.empty((M, L.O), np.uint16) for L in lins]
    lin_arr = (C.c_void_p * n)(*[L.h for L in lins])
    out_arr = (C.c_void_p * n)(*[o.ptr for o in outs])
    h = ctx.empty((M, K), np.uint16) if want_h else None
    normed = ctx.empty((M, K), np.uint16) if want_normed else None
    ctx.check(ctx._lib.orn_add_norm_gemv(ctx.h, _p(a), _p(b) if b is not None else None, _p(w), M, K, eps,
                                         lin_arr, out_arr, n, h.ptr if h else None,
                                         normed.ptr if normed else None), "orn_add_norm_gemv")
    return outs, h, normed


def generate_step(model, cache, prompt, max_tokens, prefill_step=2048, on_token=None):
    """generate::generate_step with the Greedy sampler (src/generate.rs:162-206).
    Returns the list of emitted tokens; `on_token(tok) -> bool` may stop early."""
    prompt = np.ascontiguousarray(prompt, np.uint32)
    out = []

    def cb(tok, _user):
        out.append(int(tok))
        return 1 if (on_token is None or on_token(int(tok))) else 0

    cbf = _ffi.TOKEN_CB(cb)
    rc = model.ctx._lib.orn_generate_step(model.h, cache.h, prompt.ctypes.data, len(prompt), max_tokens,
                                          prefill_step, cbf, None)
    model.ctx.check(rc, "orn_generate_step")
    return out


def generate_step_mtp(model, cache, prompt, depth, max_tokens, prefill_step=2048,
                      policy=POLICY_COMMITTED, frspec=False, force=None, on_token=None):
    """mtp_generate::generate_step_mtp (src/mtp_generate.rs:150-317).  `force` is
    (stream, p, seed): with probability p the draft for generated position i is
    replaced by stream[i].  Returns (tokens, MtpStats)."""
    prompt = np.ascontiguousarray(prompt, np.uint32)
    out = []

    def cb(tok, _user):
        out.append(int(tok))
        return 1 if (on_token is None or on_token(int(tok))) else 0

    cbf = _ffi.TOKEN_CB(cb)
    stats = MtpStats()
    fd = None
    keep = None
    if force is not None:
        stream, p, seed = force
        keep = np.ascontiguousarray(stream, np.uint32)
        fd = ForceDraft(stream=keep.ctypes.data, len=len(keep), p=p, seed=seed)
    rc = model.ctx._lib.orn_generate_step_mtp(model.h, cache.h, prompt.ctypes.data, len(prompt), depth,
                                              max_tokens, prefill_step, policy, int(bool(frspec)),
                                              C.byref(fd) if fd is not None else None, cbf, None,
                                              C.byref(stats))
    model.ctx.check(rc, "orn_generate_step_mtp")
    return out, stats
