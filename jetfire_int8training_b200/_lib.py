"""ctypes binding of the C ABI declared in include/jetfire_b200.h.

There is no CPU fallback: if the compiled library is missing, importing an operator raises, and every
operator raises on non-CUDA tensors.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libjetfire_b200.so")

_i64, _u64, _int, _vp = ctypes.c_int64, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p

# name -> argument types, exactly the prototypes of include/jetfire_b200.h
SIGNATURES = {
    "jf_status_string": ([_int], ctypes.c_char_p),
    "jf_last_cuda_error": ([], _int),
    "jf_abi_version": ([], _int),
    "jf_int8_quantize": ([_vp, _int, _i64, _i64, _vp, _vp, _vp, _int, _vp, _u64, _u64, _vp], _int),
    "jf_int8_quantize_multi": ([_int, _vp, _int, _vp, _vp, _vp, _vp, _vp], _int),
    "jf_int8_dequantize": ([_vp, _vp, _i64, _i64, _vp, _vp], _int),
    "jf_int8_transpose": ([_vp, _i64, _i64, _vp, _vp], _int),
    "jf_int8_gelu_forward": ([_vp, _vp, _i64, _i64, _vp, _vp, _vp], _int),
    "jf_int8_gelu_backward": ([_vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _int, _vp, _u64, _u64, _vp], _int),
    "jf_int8_layernorm_forward": ([_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp], _int),
    "jf_int8_layernorm_backward": ([_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _vp, _int, _vp,
                                    _u64, _u64, _vp], _int),
    "jf_int8_add": ([_vp, _int, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _int, _vp, _u64, _u64, _vp], _int),
    "jf_int8_add_meanvar": ([_vp, _int, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp], _int),
    "jf_int8_add_meanvar_noalloc": ([_vp, _int, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp], _int),
    "jf_igemm_forward": ([_vp, _vp, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp, _i64, _vp], _int),
    "jf_igemm_op16_bytes": ([_i64, _i64, _i64], _i64),
    "jf_igemm_dgrad": ([_vp, _vp, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp, _int, _vp,
                        _u64, _u64, _vp, _i64, _vp], _int),
    "jf_igemm_wgrad": ([_vp, _int, _vp, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _int, _vp, _int, _vp, _vp, _i64,
                        _vp], _int),
    "jf_igemm_wgrad_plan": ([_i64, _i64, _i64, _int], _int),
    "jf_igemm_int32": ([_vp, _vp, _i64, _i64, _i64, _vp, _vp], _int),
    "jf_igemm_error_flag": ([], _int),
    "jf_lm_loss_forward": ([_vp, _vp, _i64, _i64, _vp, _vp, _vp], _int),
    "jf_lm_loss_backward": ([_vp, _vp, _vp, _vp, ctypes.c_float, _i64, _i64, _vp], _int),
    "jf_adamw_chunk_elements": ([], _i64),
    "jf_adamw_clip_step": ([_i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, ctypes.c_double, ctypes.c_double, ctypes.c_double,
                            ctypes.c_double, ctypes.c_double, _vp, _i64, ctypes.c_double, ctypes.c_double, _vp, _vp], _int),
}

_lib = None


class JetfireError(RuntimeError):
    pass


def lib():
    """The loaded library; raises if it has not been built (python -m jetfire_int8training_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise JetfireError(
                f"{LIB_PATH} is missing: build it with `python -m jetfire_int8training_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (args, res) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = res
        _lib = L
    return _lib


def check(status, what):
    if status != 0:
        L = lib()
        msg = L.jf_status_string(status).decode()
        extra = f" (cuda error {L.jf_last_cuda_error()})" if status == -5 else ""
        raise JetfireError(f"{what}: {msg}{extra}")
