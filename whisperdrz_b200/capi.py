"""ctypes binding of libwdz.so (include/wdz.h).  Loading fails loudly when the
library has not been built: there is no CPU or eager fallback."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_lib", "libwdz.so")

WDZ_OK = 0
ERRORS = {-1: "WDZ_EINVAL", -2: "WDZ_ENOMEM", -3: "WDZ_ECUDA", -4: "WDZ_ESTATE",
          -5: "WDZ_ECAPACITY", -6: "WDZ_ENAN", -7: "WDZ_ETIMEOUT"}
WDZ_F32, WDZ_BF16 = 0, 1
FLAG_NO_TENSOR_CORE = 1
FLAG_NO_BULK_COPY = 2
FLAG_NO_GRAPH = 4
FLAG_NO_PDL = 8
FLAG_NO_CTA_PAIRS = 16
FLAG_NO_SPLIT_STEP = 32
MODE_OR, MODE_ALL_EXCEPT_TABLE, MODE_ALL_EXCEPT_RANGE, MODE_ALL = 0, 1, 2, 3
MAX_TABLES = 32
PROF_KINDS = {"cross_attn": 0, "self_attn": 1, "dec_gemm": 2, "enc_gemm": 3, "enc_attn": 4, "lm_head": 5,
              "logmel": 6}


class WdzError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{ERRORS.get(code, code)}: {msg}")
        self.code = code


class Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "n_mels", "n_audio_ctx", "n_audio_state", "n_audio_head", "n_audio_layer",
        "n_vocab", "n_text_ctx", "n_text_state", "n_text_head", "n_text_layer",
        "dtype", "n_slots", "max_tokens", "max_clips", "max_rows", "flags")]


class RuleDesc(C.Structure):
    _fields_ = [("forced_id", C.c_int32), ("mode", C.c_int32), ("arg0", C.c_int32), ("arg1", C.c_int32),
                ("table_bits", C.c_uint32), ("prefix_begin", C.c_int32), ("prefix_end", C.c_int32),
                ("n_set", C.c_int32), ("set_ids", C.c_int32 * 6), ("or_table", C.c_int32), ("allow_table", C.c_int32),
                ("n_clear", C.c_int32), ("clear_ids", C.c_int32 * 4),
                ("n_pen", C.c_int32), ("pen_ids", C.c_int32 * 10)]


assert C.sizeof(RuleDesc) == 128

# name -> (restype, argtypes); every symbol include/wdz.h declares
P, I, I64, SZ = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
SYMBOLS = {
    "wdz_engine_create": (I, [C.POINTER(Config), C.POINTER(P)]),
    "wdz_engine_destroy": (I, [P]),
    "wdz_workspace_bytes": (I, [P, C.POINTER(SZ)]),
    "wdz_set_workspace": (I, [P, P, SZ]),
    "wdz_bind": (I, [P, C.c_char_p, P, I64]),
    "wdz_finalize": (I, [P]),
    "wdz_last_error": (C.c_char_p, [P]),
    "wdz_version": (C.c_char_p, []),
    "wdz_device_status": (I, [P, P]),
    "wdz_launch_count": (I, [P, C.POINTER(I64)]),
    "wdz_profile": (I, [P, I]),
    "wdz_profile_read": (I, [P, I, C.POINTER(C.c_double), C.POINTER(I64), C.POINTER(C.c_double)]),
    "wdz_logmel": (I, [P, P, I64, P, P, I, P, P]),
    "wdz_logmel_static": (I, [P, P, I64, P, P, I, P, P]),
    "wdz_encode": (I, [P, P, I, P, P]),
    "wdz_linear": (I, [P, P, I, I, P, P, I, I, P, I, P]),
    "wdz_linear_rows": (I, [P, P, I, I, P, P, I, I, P, P]),
    "wdz_encoder_attention": (I, [P, P, I, P, I, P]),
    "wdz_cross_kv": (I, [P, P, P, I, P]),
    "wdz_slot_reset": (I, [P, P, I, P]),
    "wdz_slot_seqlens": (I, [P, P, P]),
    "wdz_forward_rows": (I, [P, P, P, P, I, P, I, P, P]),
    "wdz_prefill": (I, [P, P, P, I, P, P, P, I, P, I, P, P]),
    "wdz_decode_step": (I, [P, P, P, I, P, P, P, P]),
    "wdz_ts_configure": (I, [P, I, I, I, I, I, C.c_uint32, C.c_uint32]),
    "wdz_ts_reset": (I, [P, P, P, I, P]),
    "wdz_ts_first": (I, [P, P, P, I, P]),
    "wdz_ts_steps": (I, [P, P, I, I, P]),
    "wdz_ts_poll": (I, [P, P, P]),
    "wdz_ts_tokens": (I, [P, I, P, I, P]),
    "wdz_reargmax": (I, [P, P, P, I, P, P]),
    "wdz_rules_argmax": (I, [P, P, P, I, I, P, P]),
    "wdz_align_configure": (I, [P, P, I]),
    "wdz_align_capacity": (I, [P, I]),
    "wdz_align_matrix": (I, [P, P, P, P, P, I, I, P, P]),
    "wdz_dtw": (I, [P, P, I64, I64, P, P, P, P, P, I, I, I, I, P, P, P, P]),
}

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m whisperdrz_b200.build` "
                "(the engine has no fallback path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
