"""CPU: the C-ABI library loads and exports every symbol declared in include/*.h (no compute without a GPU), argument
validation that needs no device, and the host-side mirror of the reference's operator interface."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT


@pytest.fixture(scope="module")
def libpath():
    from jetfire_int8training_b200 import build
    return build.build()


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            src = open(os.path.join(inc, f)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            names |= set(re.findall(r"\b(jf_[a-z0-9_]+)\s*\(", src))
    return sorted(names)


def test_library_exports_every_declared_symbol(libpath):
    L = ctypes.CDLL(libpath)
    names = declared_symbols()
    assert len(names) >= 18
    for nme in names:
        assert hasattr(L, nme), f"{nme} is declared in include/ but not exported"


def test_binding_table_matches_header(libpath):
    from jetfire_int8training_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    L = _lib.lib()
    assert L.jf_abi_version() == 1
    assert b"multiples of 32" in L.jf_status_string(-2)


def test_argument_validation_needs_no_device(libpath):
    from jetfire_int8training_b200 import _lib
    L = _lib.lib()
    buf = (ctypes.c_char * 4096)()
    p = (ctypes.addressof(buf) + 15) & ~15
    assert L.jf_int8_quantize(None, 0, 32, 32, p, p, None, 0, None, 0, 0, None) == -1
    assert L.jf_int8_quantize(p, 0, 33, 32, p, p, None, 0, None, 0, 0, None) == -2
    assert L.jf_int8_quantize(p + 4, 0, 32, 32, p, p, None, 0, None, 0, 0, None) == -3
    assert L.jf_int8_quantize(p, 9, 32, 32, p, p, None, 0, None, 0, 0, None) == -4
    assert L.jf_int8_layernorm_backward(p, p, p, p, p, p, p, 32, 128, 64, p, p, p, p, 0, None, 0, 0, None) == -7
    assert L.jf_igemm_wgrad_plan(768, 768, 12288, 3) == 3
    assert L.jf_igemm_wgrad_plan(768, 768, 12288, 1) == 1
    assert L.jf_igemm_wgrad_plan(768, 768, 100, 1) == -2


def test_operators_refuse_cpu_tensors():
    from jetfire_int8training_b200 import Linear, Nonlinear
    x = torch.randn(32, 32)
    with pytest.raises(RuntimeError):
        Nonlinear.int8_quantize(x, 32)
    q = torch.zeros(32, 32, dtype=torch.int8); s = torch.ones(1, 1, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        Nonlinear.int8_gelu_forward(q, s, 32)
    with pytest.raises(RuntimeError):
        Linear.int8_linear_forward(q, s, q, s, True, 32)
    with pytest.raises(ValueError):
        Linear.int8_linear_forward(q, s, q, s, True, 16)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from jetfire_int8training_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.JetfireError):
        _lib.lib()


def test_reference_import_names():
    """The reference's callers import `Nonlinear`, `Linear` and `BlockQuantizeCUDA` as top-level modules."""
    from jetfire_int8training_b200 import compat
    compat.install()
    import Linear
    import Nonlinear
    import BlockQuantizeCUDA
    for name in ("int8_gelu_forward", "int8_gelu_backward", "int8_layernorm_forward", "int8_layernorm_backward", "int8_quantize",
                 "int8_quantize_transpose", "int8_transpose", "int8_add_Ifp_Ig16_Ofp_Og", "int8_add_Ifp_Ig16_Ofp_Og_MeanVar"):
        assert callable(getattr(Nonlinear, name))
    assert callable(Linear.int8_linear_forward) and callable(Linear.int8_linear_backward)
    for name in ("igemm_output_int_quantize_bias_rowcol", "igemm_output_int_quantize_stochastic", "igemm_output_fp_no_quantize"):
        assert callable(getattr(BlockQuantizeCUDA, name))


def test_sr_key_stream():
    from jetfire_int8training_b200 import rng
    rng.manual_seed(123, 10)
    assert rng.next_key() == (123, 10) and rng.next_key() == (123, 11)


def test_sr_noise_mode_switch():
    from jetfire_int8training_b200 import Nonlinear as NL
    prev = NL.set_sr_noise("torch")
    assert prev == "philox" and NL.set_sr_noise(prev) == "torch"
    with pytest.raises(ValueError):
        NL.set_sr_noise("curand")


def test_clip_adamw_refuses_cpu_parameters():
    """No CPU path: the optimiser step only exists as a CUDA kernel."""
    from jetfire_int8training_b200.optim import ClipAdamW
    with pytest.raises(ValueError):
        ClipAdamW([([torch.nn.Parameter(torch.zeros(8))], 0.0)], lr=1e-3)


def test_argument_validation_of_the_newer_entry_points(libpath):
    """jf_int8_quantize_multi, jf_lm_loss_* and jf_adamw_clip_step refuse bad arguments before touching a device."""
    from jetfire_int8training_b200 import _lib
    L = _lib.lib()
    buf = (ctypes.c_char * 4096)()
    p = (ctypes.addressof(buf) + 15) & ~15
    one = ctypes.c_void_p * 1
    i64 = ctypes.c_int64 * 1
    f32 = ctypes.c_float * 1
    assert L.jf_int8_quantize_multi(0, one(p), 0, i64(32), i64(32), one(p), one(p), None) == -7          # count out of 1..8
    assert L.jf_int8_quantize_multi(9, one(p), 0, i64(32), i64(32), one(p), one(p), None) == -7
    assert L.jf_int8_quantize_multi(1, one(p), 0, i64(33), i64(32), one(p), one(p), None) == -2          # not a multiple of 32
    assert L.jf_int8_quantize_multi(1, one(None), 0, i64(32), i64(32), one(p), one(p), None) == -1
    assert L.jf_lm_loss_forward(None, p, 4, 512, p, p, None) == -1
    assert L.jf_lm_loss_forward(p, p, 0, 512, p, p, None) == -2
    assert L.jf_adamw_chunk_elements() == 4096
    args = dict(lr=1e-3, b1=0.9, b2=0.95, eps=1e-8, mn=1.0)
    call = lambda n, g, numel, start, total, state=p: L.jf_adamw_clip_step(n, g, numel, start, f32(0.0), p, p, p, total, 1e-3, 0.9, 0.95,
                                                                            1e-8, 1.0, state, 2000, 2.0, 0.5, p, None)
    assert call(1, one(p), i64(4096), i64(0), 1, state=None) == -1
    assert call(0, one(p), i64(4096), i64(0), 1) == -2
    assert call(1, one(p), i64(4098), i64(0), 2) == -2                      # numel not a multiple of 4
    assert call(1, one(p), i64(8192), i64(0), 1) == -2                      # the segment does not fit its chunks
    assert call(1, one(p + 4), i64(4096), i64(0), 1) == -3                  # gradient not 16-byte aligned
    assert call(1, one(None), i64(4096), i64(0), 1) == -1
