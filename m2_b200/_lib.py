"""ctypes binding of libm2b200.so (the C ABI declared in include/m2_b200.h).

There is no fallback: if the shared library is missing or a call fails, a RuntimeError is
raised.  Build the library with ``python -m m2_b200.csrc.build``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libm2b200.so")
ABI_VERSION = 2

M2_F32, M2_BF16, M2_F16 = 0, 1, 2

c_float_p = C.POINTER(C.c_float)


class FilterArgs(C.Structure):
    _fields_ = [
        ("d_model", C.c_int), ("seq_len", C.c_int), ("order", C.c_int), ("emb_dim", C.c_int),
        ("bidirectional", C.c_int), ("bf16_rounding", C.c_int),
        ("w_mod", C.c_float), ("shift", C.c_float),
        ("z", C.c_void_p), ("t", C.c_void_p),
        ("w", C.c_void_p * 4), ("b", C.c_void_p * 3),
        ("w_rev", C.c_void_p * 4), ("b_rev", C.c_void_p * 3),
        ("freq", C.c_void_p), ("deltas", C.c_void_p), ("k_out", C.c_void_p),
    ]


class LongconvArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int), ("seq_len", C.c_int), ("d_model", C.c_int),
        ("n_filters", C.c_int), ("plain", C.c_int), ("kind", C.c_int),
        ("act_dtype", C.c_int), ("u_dtype", C.c_int), ("bf16_rounding", C.c_int),
        ("xin", C.c_void_p), ("xin_sb", C.c_longlong), ("xin_st", C.c_longlong), ("xin_sc", C.c_longlong),
        ("u", C.c_void_p), ("u_sb", C.c_longlong), ("u_st", C.c_longlong), ("u_sc", C.c_longlong),
        ("out", C.c_void_p), ("out_sb", C.c_longlong), ("out_st", C.c_longlong), ("out_sc", C.c_longlong),
        ("short_w", C.c_void_p), ("short_b", C.c_void_p),
        ("spec", C.c_void_p * 2), ("bias", C.c_void_p * 2),
        ("yu_bf16", C.c_int),
    ]


class TimeMajorArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int), ("seq_len", C.c_int), ("d_model", C.c_int), ("src_dtype", C.c_int),
        ("src", C.c_void_p), ("src_sb", C.c_longlong), ("src_st", C.c_longlong), ("src_sc", C.c_longlong),
        ("dst", C.c_void_p), ("dst_sb", C.c_longlong), ("dst_sc", C.c_longlong),
    ]


class BlockdiagArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int), ("nblocks", C.c_int), ("p", C.c_int), ("q", C.c_int),
        ("in_features", C.c_int), ("out_features", C.c_int), ("dtype", C.c_int),
        ("x", C.c_void_p), ("ldx", C.c_longlong), ("w", C.c_void_p), ("bias", C.c_void_p),
        ("out", C.c_void_p), ("ldo", C.c_longlong), ("variant", C.c_int),
    ]


class GluArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int), ("d_model", C.c_int), ("inter", C.c_int), ("nblocks", C.c_int),
        ("dtype", C.c_int),
        ("x", C.c_void_p), ("ldx", C.c_longlong), ("wg", C.c_void_p),
        ("h", C.c_void_p), ("ldh", C.c_longlong), ("variant", C.c_int),
    ]


class LinearArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int), ("seq_len", C.c_int), ("in_features", C.c_int), ("out_features", C.c_int),
        ("dtype", C.c_int),
        ("x", C.c_void_p), ("x_sb", C.c_longlong), ("x_st", C.c_longlong), ("x_sc", C.c_longlong),
        ("w", C.c_void_p), ("bias", C.c_void_p),
        ("out", C.c_void_p), ("out_sb", C.c_longlong), ("out_st", C.c_longlong), ("out_sc", C.c_longlong),
        ("force_simt", C.c_int),
    ]


class AddLayernormArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int), ("n", C.c_int), ("in_dtype", C.c_int), ("out_dtype", C.c_int),
        ("a", C.c_void_p), ("lda", C.c_longlong), ("b", C.c_void_p), ("ldb", C.c_longlong),
        ("weight", C.c_void_p), ("bias", C.c_void_p), ("eps", C.c_float),
        ("out", C.c_void_p), ("ldo", C.c_longlong),
        ("out_bf16", C.c_void_p), ("ld_bf16", C.c_longlong),
        ("out_tm_f16", C.c_void_p), ("tm_sb", C.c_longlong), ("tm_sc", C.c_longlong), ("seq_len", C.c_int),
        ("bf16_pad_cols", C.c_int),
    ]


class EmbedLayernormArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int), ("n", C.c_int),
        ("word_table", C.c_void_p), ("input_ids", C.c_void_p),
        ("type_table", C.c_void_p), ("token_type_ids", C.c_void_p),
        ("pos_table", C.c_void_p), ("position_ids", C.c_void_p),
        ("weight", C.c_void_p), ("bias", C.c_void_p), ("eps", C.c_float),
        ("out", C.c_void_p), ("ldo", C.c_longlong),
        ("out_bf16", C.c_void_p), ("ld_bf16", C.c_longlong), ("bf16_pad_cols", C.c_int),
        ("out_tm_f16", C.c_void_p), ("tm_sb", C.c_longlong), ("tm_sc", C.c_longlong), ("seq_len", C.c_int),
        ("vocab_rows", C.c_longlong), ("type_rows", C.c_longlong), ("pos_rows", C.c_longlong),
    ]


# name -> (restype, argtypes); every symbol include/m2_b200.h declares
SYMBOLS = {
    "m2_version": (C.c_int, []),
    "m2_last_error": (C.c_char_p, []),
    "m2_device_status": (C.c_int, [C.POINTER(C.c_int)]),
    "m2_selftest_wait_timeout": (C.c_int, [C.c_ulonglong, C.c_void_p]),
    "m2_filter_row_len": (C.c_int, [C.c_int]),
    "m2_hyena_filter": (C.c_int, [C.POINTER(FilterArgs), C.c_void_p]),
    "m2_longconv_kind": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "m2_filter_spectrum_floats": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "m2_filter_spectrum": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "m2_longconv_kind_batch": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "m2_filter_spectrum_bias": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "m2_linear_fwd": (C.c_int, [C.POINTER(LinearArgs), C.c_void_p]),
    "m2_longconv_fwd": (C.c_int, [C.POINTER(LongconvArgs), C.c_void_p]),
    "m2_time_major_f16": (C.c_int, [C.POINTER(TimeMajorArgs), C.c_void_p]),
    "m2_blockdiag_fwd": (C.c_int, [C.POINTER(BlockdiagArgs), C.c_void_p]),
    "m2_blockdiag_glu_fwd": (C.c_int, [C.POINTER(GluArgs), C.c_void_p]),
    "m2_add_layernorm_fwd": (C.c_int, [C.POINTER(AddLayernormArgs), C.c_void_p]),
    "m2_embed_layernorm_fwd": (C.c_int, [C.POINTER(EmbedLayernormArgs), C.c_void_p]),
}

_lib = None


def lib():
    """The loaded library; raises RuntimeError if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: the CUDA extension is not built "
                "(run `python -m m2_b200.csrc.build`); m2_b200 has no fallback path")
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(handle, name)   # AttributeError if the symbol is missing
            fn.restype = restype
            fn.argtypes = argtypes
        if handle.m2_version() != ABI_VERSION:
            raise RuntimeError(f"libm2b200.so has ABI {handle.m2_version()}, expected {ABI_VERSION}")
        _lib = handle
    return _lib


def check(rc, what=""):
    if rc != 0:
        msg = lib().m2_last_error().decode(errors="replace")
        raise RuntimeError(f"m2_b200 {what} failed (status {rc}): {msg}")
