"""The C-ABI library loads without a GPU and exports every declared symbol."""
import ctypes as C
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ornith_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(orn_[a-z0-9_]+)\s*\(", text)) - {"orn_token_cb"})


def test_every_declared_symbol_is_exported(pkg):
    lib = pkg.lib()
    names = declared_symbols()
    assert len(names) > 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    from ornith_rs_b200 import _ffi
    assert sorted(_ffi.SIGNATURES) == names


def test_host_math_equals_oracle_math(pkg):
    """The library's elementary functions (host copies) and the oracle's
    restatement agree bit for bit on every bfloat16 input."""
    import helpers as hp
    import orn_oracle as orc
    lib = pkg.lib()
    h = np.arange(0, 65536, 7, dtype=np.uint32).astype(np.uint16)
    x = hp.bf16_to_f32(h)
    x = x[np.isfinite(x)]
    xs = hp.f32_to_bf16(x)
    ones = hp.f32_to_bf16(np.ones(len(x), np.float32))
    got = np.array([lib.orn_host_sigmoid_bf(float(v)) for v in x], np.float32)
    ref = hp.bf16_to_f32(orc.sigmoid_gate(xs, ones, len(x), 1))
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    # exp / log against float64 within 2 ulp
    for v in np.linspace(-80, 80, 401, dtype=np.float32):
        e = lib.orn_host_expf(float(v))
        assert abs(e - np.exp(np.float64(v))) <= 2.5 * np.spacing(np.float32(np.exp(np.float64(v))))
    for v in np.geomspace(1e-30, 1e30, 301).astype(np.float32):
        l = lib.orn_host_logf(float(v))
        r = np.log(np.float64(v))
        assert abs(l - r) <= 3 * np.spacing(np.float32(abs(r))) + 1e-7
    s, c = C.c_float(), C.c_float()
    for a in np.linspace(0, 5000, 503, dtype=np.float32):
        lib.orn_host_sincosf(float(a), C.byref(s), C.byref(c))
        assert abs(s.value - np.sin(np.float64(a))) < 2e-6 and abs(c.value - np.cos(np.float64(a))) < 2e-6


def test_no_gpu_means_a_clean_error(pkg):
    """Without a device the context cannot be created and nothing falls back."""
    lib = pkg.lib()
    import torch
    if torch.cuda.is_available():
        return
    h = C.c_void_p()
    assert lib.orn_ctx_create(0, C.byref(h)) != 0


# --- the Rust binding text of INTEGRATION.md against the header -------------------------------
_C2RUST = {"int32_t": "i32", "uint32_t": "u32", "int64_t": "i64", "uint64_t": "u64", "size_t": "usize", "float": "f32",
           "uint16_t": "u16", "uint8_t": "u8", "void": "c_void", "char": "c_char", "orn_ctx": "OrnCtx",
           "orn_linear": "OrnLinear", "orn_model": "OrnModel", "orn_cache": "OrnCache", "orn_config": "OrnConfig",
           "orn_mtp_stats": "OrnMtpStats", "orn_force_draft": "OrnForceDraft", "orn_prof": "OrnProf",
           "orn_token_cb": "OrnTokenCb", "orn_ep": "OrnEp", "orn_batch": "OrnBatch"}


def _rust_type(ctype):
    """`const T* const*` -> `*const *const T` (pointer levels inside out, constness per level)."""
    t = re.sub(r"\s+", " ", ctype.strip())
    m = re.match(r"^(const )?([A-Za-z_0-9]+) ?((?:\* ?(?:const ?)?)*)$", t)
    assert m, ctype
    const, base, stars = m.group(1), m.group(2), m.group(3)
    r = _C2RUST[base]
    levels = re.findall(r"\*\s*(const)?", stars)
    for i in range(len(levels)):
        is_const = (const is not None) if i == 0 else (levels[i - 1] == "const")
        r = ("*const " if is_const else "*mut ") + r
    return r


def _header_prototypes():
    text = open(os.path.join(ROOT, "include", "ornith_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for ret, name, args in re.findall(r"^\s*((?:const\s+)?[A-Za-z_0-9]+\s*\*?)\s*(orn_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;",
                                      text, flags=re.M | re.S):
        if name == "orn_token_cb":
            continue
        args = re.sub(r"\s+", " ", args.strip())
        types = []
        if args and args != "void":
            for a in args.split(","):
                types.append(_rust_type(re.match(r"^(.*?)[A-Za-z_0-9]+$", a.strip()).group(1)))
        protos[name] = (types, _rust_type(ret))
    return protos


def test_rust_binding_text_matches_the_header():
    """The `extern "C"` block a maintainer would paste into the crate declares
    every entry point of the header with the same arity, argument types and return type."""
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    block = doc[doc.index('extern "C" {'):]
    block = block[:block.index("\n}")]
    block = re.sub(r"//[^\n]*", "", block)
    rust = {}
    for name, args, ret in re.findall(r"pub fn (orn_[a-z0-9_]+)\s*\(([^;]*?)\)\s*(?:->\s*([^;]+?))?\s*;", block, flags=re.S):
        types = [re.sub(r"\s+", " ", a.split(":", 1)[1].strip()) for a in args.split(",") if a.strip()]
        rust[name] = (types, (ret or "c_void").strip())
    header = _header_prototypes()
    assert sorted(rust) == sorted(header), sorted(set(rust) ^ set(header))
    for name, proto in header.items():
        assert rust[name] == proto, (name, rust[name], proto)
