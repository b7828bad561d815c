"""ctypes binding of libcbl.so (the C ABI declared in include/cbl.h).

There is no fallback: if the shared object is missing or lacks a symbol, importing this module
raises. Build it with `python -m quantexperiments_b200.build`."""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libcbl.so"

OK, EINVAL, EUNSUPPORTED, ECUDA, ETIMEOUT = 0, -1, -2, -3, -4
F32, F16, BF16 = 0, 1, 2


class CblError(RuntimeError):
    """A libcbl entry point returned a negative status."""

    def __init__(self, fn: str, status: int, detail: str):
        super().__init__(f"{fn}: {detail} (status {status})")
        self.status = status


class Packed(Structure):
    """struct cbl_packed: the file layout of one matrix, device pointers."""
    _fields_ = [("R", c_int32), ("C", c_int32), ("d", c_int32), ("bits", c_int32), ("G", c_int32), ("M", c_int32),
                ("books", c_int32), ("W", c_int32), ("tags", c_void_p), ("tags2", c_void_p), ("table", c_void_p),
                ("table2", c_void_p), ("row_scale", c_void_p), ("row_book", c_void_p), ("row_mask", c_void_p),
                ("perms", c_void_p)]


class T16(Structure):
    """struct cbl_t16: row-tile layout for the small-batch product."""
    _fields_ = [("R", c_int32), ("C", c_int32), ("books", c_int32), ("M", c_int32), ("ntile", c_int32),
                ("nsuper", c_int32), ("words", c_void_p), ("tile_rows", c_void_p), ("tile_mask", c_void_p),
                ("table", c_void_p), ("table2", c_void_p), ("row_scale", c_void_p)]


class X16(Structure):
    """struct cbl_x16: activation-stationary layout for 16..32 tokens."""
    _fields_ = [("R", c_int32), ("C", c_int32), ("books", c_int32), ("nkr", c_int32), ("nrb", c_int32),
                ("words", c_void_p), ("table", c_void_p), ("table2", c_void_p), ("row_scale", c_void_p)]


L8_MAX_ORDERS = 16


class L8(Structure):
    """struct cbl_l8: column-tile layout (rot = 1: the batch-1 product; rot = 0: the tensor-core products)."""
    _fields_ = [("R", c_int32), ("C", c_int32), ("books", c_int32), ("ntile", c_int32), ("Rpad", c_int32),
                ("rot", c_int32), ("M", c_int32), ("book_exp", c_int32),
                ("words", c_void_p), ("frag", c_void_p), ("frag2", c_void_p), ("row_scale", c_void_p),
                ("table", c_void_p), ("table2", c_void_p), ("row_index", c_void_p), ("perms", c_void_p),
                ("seg_off", c_int32 * (L8_MAX_ORDERS + 1)), ("book_exp2", c_int32)]


# name -> (restype, argtypes); every symbol include/cbl.h declares
SIGNATURES = {
    "cbl_version": (c_int, []),
    "cbl_built_for_sm": (c_int, []),
    "cbl_status_string": (c_char_p, [c_int]),
    "cbl_last_cuda_error": (c_int, []),
    "cbl_dequant": (c_int, [POINTER(Packed), c_void_p, c_int, c_int64, c_int32, c_int32, c_void_p]),
    "cbl_gemv_generic": (c_int, [POINTER(Packed), c_void_p, c_int, c_int32, c_int64, c_void_p, c_int, c_int64, c_void_p]),
    "cbl_unpack_tags": (c_int, [POINTER(Packed), c_int, c_void_p, c_void_p]),
    "cbl_assign_max_codewords": (c_int, []),
    "cbl_assign": (c_int, [c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_int, c_int32, c_void_p, c_void_p, c_void_p]),
    "cbl_pack_tags": (c_int, [c_void_p, c_int64, c_int32, c_int32, c_void_p, c_void_p]),
    "cbl_t16_bytes": (c_size_t, [c_int32, c_int32, c_int32]),
    "cbl_repack_t16": (c_int, [POINTER(Packed), c_void_p, c_int32, c_void_p, c_void_p]),
    "cbl_prep_x_bytes": (c_size_t, [c_int32, c_int32, c_int32]),
    "cbl_prep_x": (c_int, [c_void_p, c_int, c_int32, c_int32, c_int64, c_void_p, c_int32, c_void_p, c_void_p]),
    "cbl_gemv_t16": (c_int, [POINTER(T16), c_void_p, c_int32, c_void_p, c_int, c_int64, c_void_p]),
    "cbl_x16_bytes": (c_size_t, [c_int32, c_int32, c_int32]),
    "cbl_repack_x16": (c_int, [POINTER(Packed), c_void_p, c_void_p]),
    "cbl_gemv_x16_workspace_bytes": (c_size_t, [c_int32]),
    "cbl_gemv_x16": (c_int, [POINTER(X16), c_void_p, c_int32, c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "cbl_l8_bytes": (c_size_t, [c_int32, c_int32, c_int32]),
    "cbl_repack_l8": (c_int, [POINTER(Packed), c_void_p, c_void_p]),
    "cbl_l8r_bytes": (c_size_t, [c_int32, c_int32, c_int32]),
    "cbl_repack_l8r": (c_int, [POINTER(Packed), c_void_p, c_int32, c_void_p, c_void_p]),
    "cbl_book_frag_bytes": (c_size_t, []),
    "cbl_repack_book": (c_int, [c_void_p, c_void_p, c_void_p]),
    "cbl_book_norm_exp": (c_int, [c_void_p, POINTER(c_int32), c_void_p]),
    "cbl_gemv_l8_workspace_bytes": (c_size_t, [c_int32]),
    "cbl_gemv_l8": (c_int, [POINTER(L8), c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "cbl_gemv_l8_plan": (c_int, [POINTER(L8), c_int32, c_int32, c_void_p, c_void_p]),
    "cbl_gemv_l8_static_max_rows": (c_int32, []),
    "cbl_gemv_l8_static": (c_int, [POINTER(L8), c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "cbl_gemv_l8_static_status": (c_int, [c_void_p]),
    "cbl_gemm_stage_bytes": (c_size_t, [c_int32, c_int32]),
    "cbl_gemm_l8": (c_int, [POINTER(L8), c_void_p, c_int, c_int32, c_int64, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "cbl_gemm_l8_2sm": (c_int, [POINTER(L8), c_void_p, c_int, c_int32, c_int64, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "cbl_gemv_l8_multi": (c_int, [POINTER(L8), c_int32, c_void_p, c_int, POINTER(c_void_p), c_int, c_void_p, c_void_p]),
    "cbl_gemv_l8_ar_workspace_bytes": (c_size_t, [c_int32]),
    "cbl_gemv_l8_ar": (c_int, [POINTER(L8), c_void_p, c_int, c_void_p, c_int, POINTER(c_void_p), c_int32, c_int32, c_void_p]),
    "cbl_gemv_l8_ar_status": (c_int, [c_void_p, c_int32, c_void_p]),
    "cbl_gemv_l8_status": (c_int, [c_void_p, c_int32, c_void_p]),
    "cbl_gemm_rows_max_tokens": (c_int32, []),
    "cbl_gemm_rows_workspace_bytes": (c_size_t, [c_int32]),
    "cbl_gemm_rows_multi": (c_int, [POINTER(L8), c_int32, c_void_p, c_int, c_int32, c_int64, POINTER(c_void_p), c_int, c_int64, c_void_p,
                                    c_void_p, c_void_p]),
    "cbl_dense_scratch_bytes": (c_size_t, [c_int32, c_int32]),
    "cbl_decode_raw": (c_int, [POINTER(Packed), c_void_p, c_void_p]),
    "cbl_decode_raw_wide": (c_int, [POINTER(Packed), c_void_p, c_int32, c_void_p]),
    "cbl_gemm_dense": (c_int, [c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_int, c_int32, c_int64, c_void_p, c_int, c_int64, c_void_p,
                               c_void_p, c_void_p]),
    "cbl_embed_rows": (c_int, [c_void_p, c_int, c_int64, c_int32, c_void_p, c_int32, c_void_p, c_void_p]),
    "cbl_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_float, c_int32, c_int32, c_void_p, c_void_p]),
    "cbl_rope_kv": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_float,
                            c_int32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "cbl_attn_decode_workspace_bytes": (c_size_t, [c_int32, c_int32, c_int32]),
    "cbl_attn_decode_max_splits": (c_int32, []),
    "cbl_attn_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int32, c_int32, c_int32, c_int32, c_int32, c_float,
                                c_void_p, c_void_p, c_int32, c_void_p]),
    "cbl_silu_mul": (c_int, [c_void_p, c_int, c_int64, c_int32, c_int32, c_void_p, c_void_p]),
    "cbl_head_gemv_max_batch": (c_int32, []),
    "cbl_head_gemv": (c_int, [c_void_p, c_void_p, c_int, c_int32, c_int32, c_int32, c_void_p, c_int, c_int64, c_void_p]),
    "cbl_gemv_l8_silu_mul": (c_int, [POINTER(L8), c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "cbl_gemv_l8_add_norm_max_rows": (c_int32, []),
    "cbl_gemv_l8_add_norm": (c_int, [POINTER(L8), c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "cbl_gemv_l8_rope_kv": (c_int, [POINTER(L8), c_void_p, c_int, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_float, c_int32, c_void_p,
                                    c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "cbl_embed_rows_q4": (c_int, [c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_int32, c_void_p, c_void_p]),
    "cbl_head_q8_scratch_bytes": (c_size_t, [c_int32, c_int32]),
    "cbl_head_gemv_q8_max_batch": (c_int32, []),
    "cbl_head_gemv_q8": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int32, c_int32, c_int32, c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    "cbl_argmax": (c_int, [c_void_p, c_int, c_int64, c_int32, c_int32, c_void_p, c_void_p, c_void_p]),
}


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: run `python -m quantexperiments_b200.build` "
                          "(there is no CPU or PyTorch fallback for these kernels)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def check(fn: str, status: int) -> None:
    if status == OK:
        return
    detail = lib.cbl_status_string(status).decode()
    if status == ECUDA:
        detail += f" (cudaError {lib.cbl_last_cuda_error()})"
    raise CblError(fn, status, detail)
