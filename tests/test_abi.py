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
