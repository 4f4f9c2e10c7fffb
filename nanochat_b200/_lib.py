"""ctypes binding of libnckv.so (declared in include/nckv.h).

There is no fallback: if the shared library is missing or does not export a symbol the import
fails with an ImportError that says how to build it.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnckv.so")

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_i64 = ctypes.c_int64
c_float = ctypes.c_float
c_size_t = ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/nckv.h one to one
SIGNATURES = {
    "nckv_version": (c_int, []),
    "nckv_arch": (ctypes.c_char_p, []),
    "nckv_last_error": (ctypes.c_char_p, []),
    "nckv_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "nckv_read_status": (c_int, [c_void_p, c_int, c_void_p]),
    "nckv_append_rope_norm": (c_int, [c_void_p] * 9 + [c_int] * 6 + [c_i64, c_i64, c_int, c_float,
                                                             c_float, c_void_p, c_void_p]),
    "nckv_append_rope_norm_at": (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_i64, c_i64, c_int, c_float, c_float,
                                                          c_void_p, c_void_p]),
    "nckv_append_rope_norm_split": (c_int, [c_void_p] * 9 + [c_int] * 6 + [c_i64, c_i64, c_int, c_float, c_float] +
                                    [c_int] * 3 + [c_void_p, c_void_p]),
    "nckv_kv_split_plan": (c_int, [c_void_p] + [c_int] * 5 + [c_void_p, c_void_p, c_void_p]),
    "nckv_append": (c_int, [c_void_p] * 5 + [c_int] * 5 + [c_i64, c_i64, c_void_p, c_void_p]),
    "nckv_decode_step_host": (c_int, [c_void_p] * 10 + [c_int] * 5 + [c_i64, c_i64, c_int, c_float, c_float, c_int,
                                                       c_void_p, c_size_t, c_void_p]),
    "nckv_decode_attn": (c_int, [c_void_p] * 7 + [c_int] * 5 + [c_i64, c_i64] + [c_int] * 4 +
                         [c_void_p, c_size_t, c_void_p]),
    "nckv_decode_attn_static": (c_int, [c_void_p] * 7 + [c_int] * 5 + [c_i64, c_i64] + [c_int] * 4 +
                                [ctypes.POINTER(c_void_p), c_void_p]),
    "nckv_decode_attn_split": (c_int, [c_void_p] * 6 + [c_int] * 5 + [c_i64, c_i64] + [c_int] * 4 +
                               [ctypes.POINTER(c_void_p), c_void_p, c_void_p, c_size_t, c_void_p]),
    "nckv_decode_key_ranges": (c_int, [c_void_p] + [c_int] * 9 + [c_void_p] * 4),
    "nckv_lse_combine": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_i64, c_i64, c_void_p, c_void_p, c_void_p]),
    "nckv_p2p_buffer_bytes": (c_size_t, [c_int, c_int, c_int]),
    "nckv_p2p_push": (c_int, [c_void_p, c_int, c_int, ctypes.POINTER(c_void_p), c_int, c_int, c_void_p, c_void_p]),
    "nckv_p2p_wait_combine": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                      ctypes.c_uint64, c_void_p]),
    "nckv_glue_mix_norm": (c_int, [c_void_p] * 7 + [c_int] * 3 + [c_float] * 4 + [c_void_p]),
    "nckv_glue_relu_sq": (c_int, [c_void_p, c_void_p, c_i64, c_void_p]),
    "nckv_glue_ve_gate": (c_int, [c_void_p, c_i64] + [c_void_p] * 3 + [c_int] * 3 + [c_void_p]),
    "nckv_append_rope_norm_strided": (c_int, [c_void_p] * 3 + [c_i64] * 3 + [c_void_p] * 6 + [c_int] * 6 + [c_i64, c_i64, c_int, c_float, c_float,
                                              c_void_p, c_void_p]),
    "nckv_paged_tile_tokens": (c_int, []),
    "nckv_append_rope_norm_paged": (c_int, [c_void_p] * 10 + [c_int] * 8 + [c_i64, c_i64, c_int, c_float, c_float,
                                                             c_void_p, c_void_p]),
    "nckv_decode_attn_paged": (c_int, [c_void_p] * 8 + [c_int] * 7 + [c_i64, c_i64, c_int, c_int, c_void_p, c_size_t,
                                                        c_void_p]),
    "nckv_paged_fill": (c_int, [c_void_p] * 5 + [c_int] * 7 + [c_void_p]),
    "nckv_prefill_broadcast": (c_int, [c_void_p] * 5 + [c_int] * 7 + [c_void_p]),
    "nckv_prefill_attn": (c_int, [c_void_p] * 5 + [c_int] * 6 + [c_i64, c_i64, c_int, c_void_p, c_void_p]),
    "nckv_flash_attn_fwd": (c_int, [c_void_p] * 5 + [c_int] * 6 + [c_void_p, c_void_p]),
    "nckv_flash_attn_bwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "nckv_flash_attn_bwd": (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_void_p]),
}

ERROR_NAMES = {-1: "NCKV_E_ARG", -2: "NCKV_E_UNSUPPORTED", -3: "NCKV_E_CAPACITY", -4: "NCKV_E_CUDA"}
ST_OVERFLOW, ST_TIMEOUT, ST_BAD_SEQLEN, ST_BAD_PAGE = 1, 2, 4, 8


class NckvError(RuntimeError):
    """A libnckv entry point rejected its arguments or a CUDA call failed."""

    def __init__(self, fn, code, text):
        self.fn, self.code, self.text = fn, code, text
        super().__init__(f"{fn} failed with {ERROR_NAMES.get(code, code)}: {text}")


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m nanochat_b200.csrc.build` "
            "(needs nvcc; the kernels target sm_100a and there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def check(fn_name, rc):
    """Raise NckvError for a negative return code of an entry point."""
    if rc < 0:
        raise NckvError(fn_name, rc, lib.nckv_last_error().decode("utf-8", "replace"))
    return rc


def call(fn_name, *args):
    return check(fn_name, getattr(lib, fn_name)(*args))
