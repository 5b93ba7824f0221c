"""ctypes binding of libbfp8.so.  There is no fallback: without the library every op raises."""

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libbfp8.so")

OK = 0
STATUS_NONFINITE_CODE = 0x1
STATUS_BAD_SCALE = 0x2
STATUS_WAIT_TIMEOUT = 0x4
STATUS_NONFINITE_INPUT = 0x8
OUT_F32 = 0
OUT_BF16 = 1

_c = ctypes
_i64, _ptr, _int, _sz = _c.c_int64, _c.c_void_p, _c.c_int, _c.c_size_t

# name -> (restype, argtypes); must list every symbol include/bfp8.h declares
SIGNATURES = {
    "bfp8_version": (_int, []),
    "bfp8_error_string": (_c.c_char_p, [_int]),
    "bfp8_last_cuda_error": (_int, []),
    "bfp8_set_weights_at_rest": (_int, [_int]),
    "bfp8_reencode_half": (_int, [_ptr, _ptr, _i64, _ptr, _ptr, _i64, _ptr, _ptr, _ptr]),
    "bfp8_validate_e4m3": (_int, [_ptr, _i64, _ptr, _i64, _ptr, _ptr]),
    "bfp8_quant_block128_f32": (_int, [_ptr, _i64, _i64, _i64, _ptr, _i64, _ptr, _int, _ptr]),
    "bfp8_quant_act_1x128_bf16": (_int, [_ptr, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _int, _ptr, _ptr]),
    "bfp8_decode_block128": (_int, [_ptr, _i64, _i64, _i64, _ptr, _ptr, _int, _i64, _ptr]),
    "bfp8_gemm_block128_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "bfp8_gemm_block128": (_int, [_ptr, _i64, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _ptr, _int, _i64,
                                  _i64, _i64, _i64, _ptr, _sz, _ptr, _ptr]),
    "bfp8_gemm_block128_ex": (_int, [_ptr, _i64, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _ptr, _int, _i64,
                                     _i64, _i64, _i64, _ptr, _sz, _ptr, _ptr, _int, _int, _i64]),
    "bfp8_quant_act_token_bf16": (_int, [_ptr, _i64, _i64, _i64, _ptr, _i64, _ptr, _int, _ptr, _ptr]),
    "bfp8_gemm_token_channel": (_int, [_ptr, _i64, _ptr, _ptr, _i64, _ptr, _ptr, _ptr, _int, _i64,
                                       _i64, _i64, _i64, _ptr, _ptr]),
    "bfp8_gemm_block128_noalloc": (_int, [_ptr, _i64, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _ptr, _int, _i64,
                                          _i64, _i64, _i64, _ptr, _ptr]),
    "bfp8_silu_and_mul_bf16": (_int, [_ptr, _i64, _ptr, _i64, _i64, _i64, _ptr]),
    "bfp8_silu_quant_act_1x128_bf16": (_int, [_ptr, _i64, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64, _int, _ptr, _ptr]),
    "bfp8_rank_sum": (_int, [_ptr, _ptr, _i64, _int, _int, _ptr]),
    "bfp8_rank_sum_slices": (_int, [_ptr, _ptr, _i64, _int, _int, _ptr, _i64, _ptr]),
    "bfp8_gemm_block128_push": (_int, [_ptr, _i64, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _int, _int,
                                       _i64, _i64, _i64, _ptr, _sz, _ptr, _ptr]),
    "bfp8_peer_alloc": (_int, [_sz, _ptr]),
    "bfp8_peer_free": (_int, [_ptr]),
    "bfp8_peer_export": (_int, [_ptr, _ptr]),
    "bfp8_peer_open": (_int, [_ptr, _ptr]),
    "bfp8_peer_close": (_int, [_ptr]),
    "bfp8_peer_barrier": (_int, [_ptr, _int, _int, _c.c_uint32, _i64, _ptr, _ptr]),
    "bfp8_swiglu_interleave_weight": (_int, [_ptr, _i64, _ptr, _i64, _i64, _i64, _ptr]),
    "bfp8_gemm_block128_swiglu": (_int, [_ptr, _i64, _ptr, _i64, _ptr, _i64, _ptr, _ptr, _ptr, _i64,
                                         _i64, _i64, _i64, _ptr, _sz, _ptr, _ptr]),
}

_lib = None


class Bfp8Error(RuntimeError):
    pass


def load():
    """Load libbfp8.so (once) and attach signatures.  Raises if the library has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Bfp8Error(
                "libbfp8.so is missing (%s). Build it with `python -m gaudi_kernels_b200.build`; "
                "there is no CPU or PyTorch fallback." % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc, what):
    if rc != OK:
        lib = load()
        msg = lib.bfp8_error_string(rc).decode()
        extra = ""
        if rc == -5:
            extra = " (cuda error %d)" % lib.bfp8_last_cuda_error()
        raise Bfp8Error("%s failed: %s%s" % (what, msg, extra))
