"""ctypes binding of the C ABI declared in include/dabnn_b200.h.

This is plumbing only: it loads dabnn_b200/lib/libdabnn_b200.so and attaches argument types.  There
is no fallback of any kind - if the library is missing, or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "lib" / "libdabnn_b200.so"

ENGINE_AUTO, ENGINE_POPC, ENGINE_B1, ENGINE_IMMA, ENGINE_TCGEN05 = 0, 1, 2, 3, 4
BINCONV_STATIC_BYTES = 16 << 20   # DABNN_BINCONV_STATIC_BYTES
ENGINES = {"auto": ENGINE_AUTO, "popc": ENGINE_POPC, "b1": ENGINE_B1, "imma": ENGINE_IMMA, "tcgen05": ENGINE_TCGEN05}
ERROR_NAMES = {1: "ARG", 2: "SHAPE", 3: "IO", 4: "FORMAT", 5: "UNSUPPORTED", 6: "NOT_FOUND", 7: "CUDA",
               8: "OOM", 9: "STATE", 10: "TIMEOUT"}


class DabnnError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"dabnn error {code} ({ERROR_NAMES.get(code, '?')}): {text}")
        self.code = code
        self.text = text


_p, _i, _z, _f = C.c_void_p, C.c_int, C.c_size_t, C.c_float
# name -> argtypes; every function returns int unless listed in _RESTYPES
_SIGNATURES = {
    "dabnn_pack_mat": [_p, _p, _i, _i, _i, _i, _p],
    "dabnn_pack_64": [_p, _p, _z, _p],
    "dabnn_pad_bits": [_p, _p, _i, _i, _i, _i, _i, _i, _p],
    "dabnn_pad_f32": [_p, _p, _i, _i, _i, _i, _i, _i, _f, _p],
    "dabnn_im2col": [_p, _p, _i] + [_i] * 12 + [_p],
    "dabnn_fused_binarize_im2col": [_p, _p] + [_i] * 12 + [_p],
    "dabnn_bgemm": [_i, _i, _i, _p, _i, _p, _i, _p, _i, _i, _p],
    "dabnn_bconv": [_p, _p, _z, _p] + [_i] * 12 + [_p],
    "dabnn_binconv_workspace_bytes": [_i] * 10,
    "dabnn_binconv_forward": [_p, _p, _z, _p] + [_i] * 11 + [_p, _z, _i, _p],
    "dabnn_binconv_forward_static": [_p, _p, _z, _p] + [_i] * 11 + [_i, _p],
    "dabnn_bconv_block": [_p, _p, _z, _p, _p, _p, _p, _p] + [_i] * 12 + [_p],
    "dabnn_binarize_u8": [_p, _p, _z, _p],
    "dabnn_bconv_u8_supported": [_i] * 11,
    "dabnn_bconv_u8_weight_bytes": [_i, _i],
    "dabnn_bconv_u8_expand_weights": [_p, _z, _i, _i, _p, _p],
    "dabnn_bconv_u8_block": [_p, _p, _p, _p, _p, _p, _p, _p] + [_i] * 11 + [_p],
    "dabnn_bconv_u8_block_pooled_supported": [_i] * 11,
    "dabnn_bconv_u8_block_pooled": [_p, _p, _p, _p, _p, _p, _p, _p, _p] + [_i] * 11 + [_p],
    "dabnn_affine": [_p, _p, _p, _z, _i, _p],
    "dabnn_add": [_p, _p, _z, _p],
    "dabnn_relu": [_p, _z, _p],
    "dabnn_prelu": [_p, _p, _i, _z, _i, _p],
    "dabnn_maxpool": [_p, _p] + [_i] * 10 + [_p],
    "dabnn_avepool": [_p, _p] + [_i] * 10 + [_p],
    "dabnn_concat": [_p, _i, _p, _i, _p, _z, _p],
    "dabnn_fconv": [_p, _p, _p, _p] + [_i] * 13 + [_p],
    "dabnn_fconv_maxpool_supported": [_i] * 11,
    "dabnn_fconv_maxpool": [_p, _p, _p, _p, _p, _i, _p, _p] + [_i] * 11 + [_p],
    "dabnn_net_create": [C.POINTER(_p)],
    "dabnn_net_destroy": [_p],
    "dabnn_net_set_flags": [_p, _i, _i, _i],
    "dabnn_net_configure": [_p, _i, _i],
    "dabnn_net_read_file": [_p, C.c_char_p],
    "dabnn_net_read_buf": [_p, _p, _z],
    "dabnn_net_run": [_p, _p, _i, _i],
    "dabnn_net_sync": [_p],
    "dabnn_net_get_blob": [_p, C.c_char_p, C.POINTER(_i), C.POINTER(_p), _p, _z],
    "dabnn_net_get_blob_bits": [_p, C.c_char_p, C.POINTER(_i), C.POINTER(_p), _p, _z],
    "dabnn_net_output_name": [_p, _i],
    "dabnn_net_stream": [_p],
    "dabnn_net_stats": [_p, C.POINTER(_i), C.POINTER(_z)],
    "dabnn_net_set_host_chunk": [_p, _i],
    "dabnn_net_submit": [_p, _p, _i, C.c_char_p, _p, C.c_size_t, C.POINTER(_i)],
    "dabnn_net_wait": [_p, _i],
    "dabnn_net_set_profiling": [_p, _i],
    "dabnn_net_layer_times": [_p, C.POINTER(C.c_char_p), C.POINTER(_f), _i, C.POINTER(_i)],
    "dabnn_measure_engine_peak": [_i, C.POINTER(C.c_double)],
    "dabnn_measure_tf32_peak": [C.POINTER(C.c_double)],
    "dabnn_engine_status": [C.POINTER(_i)],
    "dabnn_last_engine": [],
    "dabnn_debug_raise_engine_status": [_i, _i],
    "dabnn_debug_set_halo": [_i],
    "dabnn_debug_set_launch_overlap": [_i],
    "dabnn_last_error": [],
    "dabnn_version": [],
    "dabnn_device_count": [],
}
_RESTYPES = {"dabnn_last_error": C.c_char_p, "dabnn_version": C.c_char_p, "dabnn_net_destroy": None,
             "dabnn_binconv_workspace_bytes": C.c_size_t, "dabnn_bconv_u8_weight_bytes": C.c_size_t, "dabnn_net_output_name": C.c_char_p,
             "dabnn_net_stream": C.c_void_p}

_lib = None


def declared_symbols():
    return sorted(_SIGNATURES)


def load():
    """Load the library (once).  Raises FileNotFoundError when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m dabnn_b200.build` (there is no CPU fallback)")
        lib = C.CDLL(str(LIB_PATH))
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _RESTYPES.get(name, C.c_int)
        _lib = lib
    return _lib


def check(rc):
    if rc != 0:
        raise DabnnError(rc, load().dabnn_last_error().decode())
