"""ctypes binding of libintfa.so (the C ABI declared in include/intfa.h).

There is no fallback: if the library has not been built, loading raises.
"""
import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libintfa.so")

OK = 0
ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE_WAIT, ERR_TOO_LARGE = -1, -2, -3, -4, -5
VARIANT_FULL, VARIANT_HALF, VARIANT_HALF_FP8 = 0, 1, 2
VSCALE_PER_TENSOR, VSCALE_PER_CHANNEL = 0, 1

EXPORTS = ("intfa_version", "intfa_last_error", "intfa_fwd", "intfa_quant_pertoken",
           "intfa_quant_v_workspace_bytes", "intfa_quant_v", "intfa_quant_qkv_workspace_bytes", "intfa_quant_qkv",
           "intfa_v_colmax", "intfa_v_quant_from_colmax", "intfa_quant_v_static",
           "intfa_quant_v_static_max_words", "intfa_scales_f16_to_f32", "intfa_sm_count")

_i64x3 = ctypes.c_int64 * 3
_i64x2 = ctypes.c_int64 * 2


class IntfaFwdParams(ctypes.Structure):
    """Mirror of `struct IntfaFwdParams` (include/intfa.h); field order and types must match."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("q_scale", ctypes.c_void_p), ("k_scale", ctypes.c_void_p), ("v_scale", ctypes.c_void_p),
        ("q_stride", _i64x3), ("k_stride", _i64x3), ("v_stride", _i64x3), ("o_stride", _i64x3),
        ("qs_stride", _i64x2), ("ks_stride", _i64x2), ("vs_stride", _i64x3),
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("Nq", ctypes.c_int32), ("Nk", ctypes.c_int32),
        ("D", ctypes.c_int32),
        ("variant", ctypes.c_int32), ("causal", ctypes.c_int32), ("sm_scale", ctypes.c_float),
        ("G", ctypes.c_int32), ("p_round", ctypes.c_int32),
        ("q_offset", ctypes.c_int64), ("kv_offset", ctypes.c_int64),
        ("lse_out", ctypes.c_void_p),
        ("state_m", ctypes.c_void_p), ("state_l", ctypes.c_void_p), ("state_acc", ctypes.c_void_p),
        ("state_in", ctypes.c_int32), ("state_out", ctypes.c_int32), ("write_o", ctypes.c_int32),
        ("dbg_s", ctypes.c_void_p), ("dbg_p", ctypes.c_void_p),
        ("dbg_tile", ctypes.c_int32), ("dbg_step", ctypes.c_int32),
        ("status", ctypes.c_void_p),
        ("H_kv", ctypes.c_int32), ("o_dtype", ctypes.c_int32),
        ("kv_order", ctypes.c_int32), ("vs_stride_blk", ctypes.c_int64),
        ("debug_wait_limit_kcycles", ctypes.c_int32), ("debug_skip_k_load", ctypes.c_int32),
    ]


class IntfaError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("libintfa error %d: %s" % (code, msg))
        self.code = code


_lib = None


def load():
    """Load libintfa.so once and declare the signatures.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libintfa.so is not built (%s missing). Build it with "
            "`python int-flashattention_b200/build.py`; there is no non-CUDA fallback." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    lib.intfa_version.restype = ctypes.c_int
    lib.intfa_version.argtypes = []
    lib.intfa_last_error.restype = ctypes.c_int
    lib.intfa_last_error.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    lib.intfa_fwd.restype = ctypes.c_int
    lib.intfa_fwd.argtypes = [ctypes.POINTER(IntfaFwdParams), vp]
    lib.intfa_quant_pertoken.restype = ctypes.c_int
    lib.intfa_quant_pertoken.argtypes = [vp, ctypes.POINTER(i64), vp, vp, i32, i32, i32, i32, vp]
    lib.intfa_quant_v_workspace_bytes.restype = ctypes.c_size_t
    lib.intfa_quant_v_workspace_bytes.argtypes = [i32, i32, i32]
    lib.intfa_quant_v.restype = ctypes.c_int
    lib.intfa_quant_v.argtypes = [vp, ctypes.POINTER(i64), vp, vp, i32, i32, i32, i32, i32, vp, ctypes.c_size_t, vp]
    lib.intfa_quant_qkv_workspace_bytes.restype = ctypes.c_size_t
    lib.intfa_quant_qkv_workspace_bytes.argtypes = [i32, i32, i32, i32]
    lib.intfa_quant_qkv.restype = ctypes.c_int
    lib.intfa_quant_qkv.argtypes = [vp, vp, vp, ctypes.POINTER(i64), vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32,
                                    vp, ctypes.c_size_t, vp]
    lib.intfa_v_colmax.restype = ctypes.c_int
    lib.intfa_v_colmax.argtypes = [vp, ctypes.POINTER(i64), vp, i32, i32, i32, i32, vp]
    lib.intfa_v_quant_from_colmax.restype = ctypes.c_int
    lib.intfa_v_quant_from_colmax.argtypes = [vp, ctypes.POINTER(i64), vp, vp, vp, i32, i32, i32, i32, i32, vp]
    lib.intfa_quant_v_static.restype = ctypes.c_int
    lib.intfa_quant_v_static.argtypes = [vp, ctypes.POINTER(i64), vp, vp, i32, i32, i32, i32, i32, vp]
    lib.intfa_quant_v_static_max_words.restype = ctypes.c_size_t
    lib.intfa_quant_v_static_max_words.argtypes = []
    lib.intfa_scales_f16_to_f32.restype = ctypes.c_int
    lib.intfa_scales_f16_to_f32.argtypes = [vp, vp, i64, vp]
    lib.intfa_sm_count.restype = ctypes.c_int
    lib.intfa_sm_count.argtypes = []
    _lib = lib
    return lib


def last_error():
    buf = ctypes.create_string_buffer(512)
    load().intfa_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(rc):
    if rc != OK:
        raise IntfaError(rc, last_error())
