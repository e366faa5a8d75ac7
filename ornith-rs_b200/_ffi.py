"""ctypes binding of libornith_cuda.so (the C ABI declared in include/ornith_cuda.h).

This is the stub a host-language binding mirrors: plain pointers and sizes, no
torch types.  The library must be present; there is no CPU fallback.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("ORN_CUDA_LIB") or os.path.join(_HERE, "libornith_cuda.so")  # the override serves A/B timing of builds

Q4K, Q6K, A8, BF16, A4 = 0, 1, 2, 3, 4
POLICY_CYCLE, POLICY_COMMITTED = 0, 1

c_void_pp = C.POINTER(C.c_void_p)
u16p = C.c_void_p
u32p = C.c_void_p
f32p = C.c_void_p


class Config(C.Structure):
    """orn_config: src/model/config.rs:9-158 of the reference."""

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


class MtpStats(C.Structure):
    _fields_ = [("cycles", C.c_int32), ("drafted", C.c_int32), ("accepted", C.c_int32),
                ("reached_by_depth", C.c_int32 * 8), ("accepted_by_depth", C.c_int32 * 8)]


class ForceDraft(C.Structure):
    _fields_ = [("stream", C.c_void_p), ("len", C.c_int32), ("p", C.c_float), ("seed", C.c_uint64)]


class Prof(C.Structure):
    _fields_ = [("prefill_ms", C.c_float), ("draft_ms", C.c_float), ("verify_ms", C.c_float),
                ("head_ms", C.c_float), ("total_ms", C.c_float), ("kernel_launches", C.c_int64),
                ("verify_steps", C.c_int64), ("draft_steps", C.c_int64), ("ar_steps", C.c_int64)]


TOKEN_CB = C.CFUNCTYPE(C.c_int32, C.c_uint32, C.c_void_p)

i32, f32, sz, u64, vp = C.c_int32, C.c_float, C.c_size_t, C.c_uint64, C.c_void_p

# name -> (restype, argtypes)
SIGNATURES = {
    "orn_ctx_create": (i32, [i32, c_void_pp]),
    "orn_ctx_destroy": (i32, [vp]),
    "orn_sync": (i32, [vp]),
    "orn_last_error": (C.c_char_p, [vp]),
    "orn_alloc": (i32, [vp, sz, c_void_pp]),
    "orn_free": (i32, [vp, vp]),
    "orn_ctx_stream": (i32, [vp, C.POINTER(vp)]),
    "orn_ctx_launches": (i32, [vp, C.POINTER(C.c_int64)]),
    "orn_memset": (i32, [vp, vp, i32, sz]),
    "orn_upload": (i32, [vp, vp, vp, sz]),
    "orn_download": (i32, [vp, vp, vp, sz]),
    "orn_linear_create": (i32, [vp, i32, i32, i32, i32, vp, vp, vp, c_void_pp]),
    "orn_linear_create_random": (i32, [vp, i32, i32, i32, i32, u64, f32, c_void_pp]),
    "orn_linear_export": (i32, [vp, vp, vp, vp, vp]),
    "orn_linear_sizes": (i32, [vp, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)]),
    "orn_linear_info": (i32, [vp] + [C.POINTER(i32)] * 4),
    "orn_debug_wait_probe": (i32, [vp, C.c_uint32]),
    "orn_ctx_ktime_begin": (i32, [vp]),
    "orn_ctx_ktime_end": (i32, [vp, C.c_char_p, sz]),
    "orn_timer_start": (i32, [vp]),
    "orn_timer_stop": (i32, [vp, C.POINTER(f32)]),
    "orn_linear_destroy": (i32, [vp, vp]),
    "orn_linear_gather_rows": (i32, [vp, vp, vp, i32, c_void_pp]),
    "orn_kq_dequantize": (i32, [vp, vp, i32, vp]),
    "orn_gemv": (i32, [vp, vp, vp, i32, vp, i32]),
    "orn_gather_gemv": (i32, [vp, vp, vp, vp, vp, i32, vp]),
    "orn_gemm": (i32, [vp, vp, vp, i32, vp, i32]),
    "orn_gemm_multi": (i32, [vp, vp, i32, vp, i32, vp, i32]),
    "orn_gather_gemm": (i32, [vp, vp, vp, vp, vp, i32, vp, i32]),
    "orn_embedding": (i32, [vp, vp, vp, i32, vp]),
    "orn_rms_norm": (i32, [vp, vp, vp, i32, i32, f32, vp]),
    "orn_add_rms_norm": (i32, [vp, vp, vp, vp, i32, i32, f32, vp, vp]),
    "orn_add_norm_gemv": (i32, [vp, vp, vp, vp, i32, i32, f32, vp, vp, i32, vp, vp]),
    "orn_rms_norm_gated": (i32, [vp, vp, vp, vp, i32, i32, f32, vp]),
    "orn_sigmoid_gate": (i32, [vp, vp, vp, i32, i32, vp]),
    "orn_swiglu": (i32, [vp, vp, vp, i32, vp]),
    "orn_softmax_precise": (i32, [vp, vp, i32, i32, vp]),
    "orn_router_topk": (i32, [vp, vp, i32, i32, i32, vp, vp]),
    "orn_moe_combine": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "orn_moe_block": (i32, [vp] + [vp] * 8 + [vp, i32, i32, i32, vp, vp]),
    "orn_ep_unique_id": (i32, [vp]),
    "orn_ep_init": (i32, [vp, vp, i32, i32, i32, c_void_pp]),
    "orn_ep_destroy": (i32, [vp]),
    "orn_ep_moe_block": (i32, [vp] + [vp] * 8 + [vp, i32, i32, i32, vp, vp]),
    "orn_ep_world": (i32, [vp]),
    "orn_ep_rank": (i32, [vp]),
    "orn_ep_peer_windows": (i32, [vp]),
    "orn_debug_ep_wait_probe": (i32, [vp]),
    "orn_batch_create": (i32, [vp, i32, i32, i32, i32, c_void_pp]),
    "orn_batch_destroy": (i32, [vp]),
    "orn_batch_reset": (i32, [vp]),
    "orn_batch_fill_random": (i32, [vp, i32, u64]),
    "orn_batch_positions": (i32, [vp, vp]),
    "orn_batch_forward": (i32, [vp, vp, vp, i32, vp, vp]),
    "orn_batch_commit": (i32, [vp, vp]),
    "orn_batch_mtp_draft": (i32, [vp, vp, vp, vp]),
    "orn_gdn_front": (i32, [vp] + [vp] * 7 + [i32] * 5 + [f32] + [vp] * 6),
    "orn_gated_delta": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp]),
    "orn_gated_delta_prefill": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp]),
    "orn_rope": (i32, [vp, vp, i32, i32, i32, i32, f32, i32]),
    "orn_sdpa_decode": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp]),
    "orn_sdpa_prefill": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp]),
    "orn_greedy": (i32, [vp, vp, i32, i32, i32, vp]),
    "orn_greedy_static": (i32, [vp, vp, i32, i32, i32, vp]),
    "orn_model_create": (i32, [vp, C.POINTER(Config), c_void_pp]),
    "orn_model_destroy": (i32, [vp]),
    "orn_model_set_linear": (i32, [vp, C.c_char_p, vp]),
    "orn_model_set_tensor": (i32, [vp, C.c_char_p, vp, sz]),
    "orn_model_init_random": (i32, [vp, u64]),
    "orn_model_load": (i32, [vp, C.c_char_p, i32, c_void_pp]),
    "orn_model_get_linear": (i32, [vp, C.c_char_p, c_void_pp]),
    "orn_model_get_tensor": (i32, [vp, C.c_char_p, c_void_pp, C.POINTER(sz)]),
    "orn_model_config": (i32, [vp, C.POINTER(Config)]),
    "orn_model_weight_bytes": (sz, [vp]),
    "orn_frspec_load": (i32, [vp, C.c_char_p]),
    "orn_frspec_set": (i32, [vp, vp, i32]),
    "orn_cache_create": (i32, [vp, c_void_pp]),
    "orn_cache_destroy": (i32, [vp]),
    "orn_cache_reset": (i32, [vp]),
    "orn_cache_offset": (i32, [vp]),
    "orn_forward": (i32, [vp, vp, vp, i32, vp, vp]),
    "orn_forward_capture": (i32, [vp, vp, vp, i32, vp]),
    "orn_prefill": (i32, [vp, vp, vp, i32, i32, vp]),
    "orn_cache_rewind": (i32, [vp, i32]),
    "orn_mtp_forward": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "orn_cache_mtp_offset": (i32, [vp]),
    "orn_cache_set_mtp_offset": (i32, [vp, i32]),
    "orn_head_greedy": (i32, [vp, vp, i32, vp, vp]),
    "orn_generate_step": (i32, [vp, vp, vp, i32, i32, i32, TOKEN_CB, vp]),
    "orn_generate_step_mtp": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32, C.POINTER(ForceDraft),
                                    TOKEN_CB, vp, C.POINTER(MtpStats)]),
    "orn_get_prof": (i32, [vp, C.POINTER(Prof)]),
    "orn_host_expf": (f32, [f32]),
    "orn_host_logf": (f32, [f32]),
    "orn_host_log1pf": (f32, [f32]),
    "orn_host_sincosf": (None, [f32, C.POINTER(f32), C.POINTER(f32)]),
    "orn_host_sigmoid_bf": (f32, [f32]),
    "orn_host_softplus_bf": (f32, [f32]),
}

_lib = None


def load():
    """Load the CUDA library; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libornith_cuda.so is missing: build it with `python ornith-rs_b200/build.py` "
            "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
