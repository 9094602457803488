"""ctypes binding of libktk.so (the C ABI declared in include/ktk.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libktk.so"

KTK_F32, KTK_BF16 = 0, 1
VARIANT_AUTO, VARIANT_SIMT, VARIANT_MMA, VARIANT_UMMA = 0, 1, 2, 3
ALLREDUCE_AUTO, ALLREDUCE_MULTICAST, ALLREDUCE_PEER = 0, 1, 2
EXCHANGE_ALLREDUCE_NORM, EXCHANGE_ALLREDUCE, EXCHANGE_SCATTER = 0, 1, 2
KTK_OK, KTK_ERR_ARG, KTK_ERR_UNSUPPORTED, KTK_ERR_WORKSPACE, KTK_ERR_CUDA, KTK_ERR_TOO_LARGE = 0, -1, -2, -3, -4, -5
STATUS_TEXT = {0: "ok", 1: "physical page id outside the cache", 2: "malformed page table",
               3: "a bounded wait on an asynchronous copy gave up",
               4: "a kernel's own consistency check failed"}


class KtkError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"libktk error {code}: {text}")
        self.code = code


class Shape(ctypes.Structure):
    _fields_ = [
        ("batch", c_int32), ("num_kv_heads", c_int32), ("group_size", c_int32),
        ("head_dim", c_int32), ("page_size", c_int32), ("dtype", c_int32),
        ("num_pages", c_int64),
    ]


class View(ctypes.Structure):
    _fields_ = [("sink_tokens", c_int32), ("local_tokens", c_int32), ("page_count", c_void_p),
                ("slot_index", c_void_p), ("seq_order", c_void_p)]


_i32p = c_void_p   # device pointers travel as integers
_SIGNATURES = {
    "ktk_last_error": (c_char_p, []),
    "ktk_version": (c_char_p, []),
    "ktk_append": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, _i32p, _i32p, _i32p,
                             POINTER(Shape), _i32p, c_void_p]),
    "ktk_build_summaries": (c_int32, [c_void_p, c_void_p, c_int64, _i32p, _i32p, _i32p, POINTER(Shape),
                                      _i32p, c_void_p]),
    "ktk_select": (c_int32, [c_void_p, c_void_p, c_int64, _i32p, _i32p, _i32p, c_int32, _i32p, _i32p,
                             c_void_p, POINTER(Shape), _i32p, c_void_p]),
    "ktk_decode_num_splits": (c_int32, [POINTER(Shape), c_int32]),
    "ktk_decode_workspace_bytes": (c_size_t, [POINTER(Shape), c_int32]),
    "ktk_sparse_decode": (c_int32, [c_void_p, c_void_p, _i32p, c_int32, _i32p, _i32p, c_float, c_void_p,
                                    c_void_p, c_size_t, c_int32, c_int32, POINTER(Shape), _i32p, c_void_p]),
    "ktk_noalloc_scratch_bytes": (c_size_t, []),
    "ktk_sparse_decode_noalloc": (c_int32, [c_void_p, c_void_p, _i32p, c_int32, _i32p, _i32p, c_float, c_void_p,
                                            c_int32, c_int32, POINTER(Shape), _i32p, c_void_p]),
    "ktk_dense_decode": (c_int32, [c_void_p, c_void_p, _i32p, _i32p, _i32p, c_int32, c_float, c_void_p,
                                   c_void_p, c_size_t, c_int32, c_int32, POINTER(Shape), _i32p, c_void_p]),
    "ktk_view_row_width": (c_int32, [c_int32, POINTER(View)]),
    "ktk_append_v": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, _i32p, _i32p, _i32p, POINTER(View),
                               POINTER(Shape), _i32p, c_void_p]),
    "ktk_append_tokens": (c_int32, [c_void_p, c_void_p, _i32p, c_int64, c_void_p, c_void_p, c_int64, _i32p, _i32p,
                                    _i32p, POINTER(View), POINTER(Shape), _i32p, c_void_p]),
    "ktk_prefill_workspace_bytes": (c_size_t, [c_int64, c_int32, c_int32]),
    "ktk_prefill_attention": (c_int32, [c_void_p, _i32p, c_int64, c_int32, c_void_p, _i32p, _i32p, _i32p,
                                        POINTER(View), c_float, c_void_p, c_void_p, c_size_t, c_int32,
                                        POINTER(Shape), _i32p, c_void_p]),
    "ktk_build_summaries_v": (c_int32, [c_void_p, c_void_p, c_int64, _i32p, _i32p, _i32p, POINTER(View),
                                        POINTER(Shape), _i32p, c_void_p]),
    "ktk_select_v": (c_int32, [c_void_p, c_void_p, c_int64, _i32p, _i32p, _i32p, c_int32, POINTER(View), c_int32,
                               _i32p, _i32p, c_void_p, POINTER(Shape), _i32p, c_void_p]),
    "ktk_sparse_decode_v": (c_int32, [c_void_p, c_void_p, _i32p, c_int32, POINTER(View), c_int32, _i32p, _i32p,
                                      c_float, c_void_p, c_void_p, c_size_t, c_int32, c_int32, POINTER(Shape),
                                      _i32p, c_void_p]),
    "ktk_dense_decode_v": (c_int32, [c_void_p, c_void_p, _i32p, _i32p, _i32p, POINTER(View), c_int32, c_float,
                                     c_void_p, c_void_p, c_size_t, c_int32, c_int32, POINTER(Shape), _i32p,
                                     c_void_p]),
    "ktk_rmsnorm": (c_int32, [c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int32, c_int32, c_void_p]),
    "ktk_add_rmsnorm": (c_int32, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int64, c_int32,
                                  c_int32, c_void_p]),
    "ktk_qkv_norm": (c_int32, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int64, c_int32,
                               c_int32, c_int32, c_void_p]),
    "ktk_allreduce_grid": (c_int32, [c_int64, c_int32]),
    "ktk_allreduce_add_rmsnorm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int64, c_int32, c_float, c_int32, _i32p, c_void_p]),
    "ktk_exchange_grid": (c_int32, [c_int64, c_int32]),
    "ktk_exchange_rows": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int64, c_int32, c_float,
                                    c_int32, c_int32, _i32p, c_void_p]),
    "ktk_rank_barrier": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, _i32p, c_void_p]),
    "ktk_copy_to_cache": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int64, c_int64,
                                    c_int32, c_int64, c_int64, c_int32, _i32p, c_void_p]),
    "ktk_qk": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int64,
                         c_int64, c_int32, c_int32, c_int32, _i32p, c_void_p]),
    "ktk_block_topk_mask": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int64, c_int32, c_int32,
                                      c_int32, _i32p, c_void_p]),
    "ktk_softmax_rows": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int64, c_void_p]),
    "ktk_sv": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int64,
                         c_int64, c_int32, c_int32, _i32p, c_void_p]),
    "ktk_token_topk_mask": (c_int32, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int64, c_int32, c_int32,
                                      c_int32, _i32p, c_void_p]),
    "ktk_paged_qk": (c_int32, [c_void_p, c_void_p, _i32p, _i32p, _i32p, POINTER(View), c_float, c_void_p, c_int64,
                               POINTER(Shape), _i32p, c_void_p]),
    "ktk_paged_sv": (c_int32, [c_void_p, _i32p, _i32p, _i32p, POINTER(View), c_void_p, c_int64, c_void_p,
                               POINTER(Shape), _i32p, c_void_p]),
    "ktk_qkv_norm_rope": (c_int32, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_int64,
                                    c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int32, c_void_p]),
    "ktk_pool_create": (c_void_p, [c_int64, c_int32, c_int32]),
    "ktk_pool_destroy": (None, [c_void_p]),
    "ktk_pool_free_pages": (c_int64, [c_void_p]),
    "ktk_pool_slot_tokens": (c_int64, [c_void_p, c_int32]),
    "ktk_pool_slot_pages": (c_int64, [c_void_p, c_int32]),
    "ktk_pool_admit": (c_int32, [c_void_p, c_int32, c_int64, c_int64]),
    "ktk_pool_extend": (c_int32, [c_void_p, c_void_p, c_int32, c_int32]),
    "ktk_pool_release": (c_int32, [c_void_p, c_int32]),
    "ktk_pool_export": (c_int64, [c_void_p, c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_void_p]),
    "ktk_silu_mul": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
    "ktk_silu_mul_rows": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32, c_void_p]),
}

#: every symbol include/ktk.h declares
EXPORTED = tuple(_SIGNATURES)

_lib = None


def load() -> ctypes.CDLL:
    """Load libktk.so, binding argument types.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python kinetics_b200/build.py` "
                "(nvcc, sm_100a).  There is no CPU or PyTorch fallback for this path.")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise KtkError(rc, load().ktk_last_error().decode())
