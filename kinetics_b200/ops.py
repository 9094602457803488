"""Operator surface of the block top-k paged decode path.

Functional wrappers over the C ABI (``include/ktk.h``) on CUDA tensors, and the torch
custom ops the reference's decoder layers call:

* ``mylib::update_kv``, ``mylib::decode``, ``mylib::qk_norm``, ``mylib::layer_norm`` -- the
  names and schemas of ``benchmark/blocktopk_decoder.py:23-85,171-184`` (same in
  ``benchmark/dense_decoder.py:21-83``), registered ONCE at import (the reference defines
  ``mylib::decode`` inside ``__init__``, so a second layer in one process raises).
* ``ktk::select_pages``, ``ktk::sparse_decode``, ``ktk::dense_decode``,
  ``ktk::append_kv_with_summary`` -- explicit-argument forms.

Every op runs a hand-written CUDA kernel from ``libktk.so`` on the current stream.  There is
no CPU implementation and no PyTorch fallback: a CPU tensor raises.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import _lib
from ._lib import Shape, check

HEAD_DIM = 128
PAGE_SIZE = 16
SPLITS_BALANCED = -1     # KTK_SPLITS_BALANCED: the library's policy for bf16 (see include/ktk.h)
VARIANT_SIMT = 1

_LAUNCHES = 0


def launch_count() -> int:
    """Kernels of libktk.so launched from this process so far."""
    return _LAUNCHES


def _launched(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.KTK_BF16
    if t.dtype == torch.float32:
        return _lib.KTK_F32
    raise TypeError(f"kinetics_b200: dtype {t.dtype} not supported (float32 or bfloat16)")


def _cuda(*ts):
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("kinetics_b200 ops need CUDA tensors: this path has no CPU fallback")
        if not t.is_contiguous():
            raise RuntimeError("kinetics_b200 ops need contiguous tensors")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _shape(batch: int, kv_cache: torch.Tensor, num_q_heads: int) -> Shape:
    if kv_cache.dim() != 5 or kv_cache.shape[1] != 2:
        raise ValueError("kv_cache must be [num_pages, 2, page_size, num_kv_heads, head_dim]")
    hkv = kv_cache.shape[3]
    if num_q_heads % hkv:
        raise ValueError(f"{num_q_heads} query heads do not divide into {hkv} kv heads")
    return Shape(batch, hkv, num_q_heads // hkv, kv_cache.shape[4], kv_cache.shape[2], _dtype_code(kv_cache),
                 kv_cache.shape[0])


class PageView:
    """How the pages of a sequence split into always-attended and scored ones (`ktk_view` in ktk.h).

    The default (no view) is the reference benchmark's: every full page in front of the page being
    filled is scored, that last page is always attended.  LiteSys semantics
    (litesys/attention/sparsity_utils.py:24-47) are ``PageView(sink_tokens=4, local_tokens=attn_local)``
    over a page table whose logical page 0 holds the 4 sink tokens.
    """

    def __init__(self, sink_tokens: int = 0, local_tokens: int = 1, page_count=None, slot_index=None,
                 seq_order=None):
        self.sink_tokens, self.local_tokens = int(sink_tokens), int(local_tokens)
        self.page_count, self.slot_index = page_count, slot_index
        # selection only: the sequences from the longest to the shortest (a permutation of 0..B-1); the
        # persistent CTAs of the selection kernel then share a ragged batch evenly
        self.seq_order = seq_order
        for t in (page_count, slot_index, seq_order):
            if t is not None and (t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous()):
                raise ValueError("PageView: page_count / slot_index / seq_order must be contiguous int32 CUDA tensors")

    def c(self):
        return _lib.View(self.sink_tokens, self.local_tokens,
                         0 if self.page_count is None else self.page_count.data_ptr(),
                         0 if self.slot_index is None else self.slot_index.data_ptr(),
                         0 if self.seq_order is None else self.seq_order.data_ptr())

    def row_width(self, topk: int) -> int:
        v = self.c()
        w = int(_lib.load().ktk_view_row_width(topk, ctypes.byref(v)))
        if w < 0:
            raise ValueError(_lib.load().ktk_last_error().decode())
        return w

    def batch(self, kv_indptr) -> int:
        return kv_indptr.numel() if self.page_count is not None else kv_indptr.numel() - 1


def _view_ref(view):
    """(ctypes pointer or None, keep-alive object)"""
    if view is None:
        return None, None
    cv = view.c()
    return ctypes.byref(cv), cv


def _batch_of(kv_indptr, view) -> int:
    return view.batch(kv_indptr) if view is not None else kv_indptr.numel() - 1


def new_status(device) -> torch.Tensor:
    """Device status word the kernels report table / page-id faults into (0 = ok)."""
    return torch.zeros(1, dtype=torch.int32, device=device)


def raise_on_status(status: torch.Tensor) -> None:
    """Synchronising check of a status word."""
    code = int(status.item())
    if code:
        raise RuntimeError(f"kinetics_b200 device status {code}: {_lib.STATUS_TEXT.get(code, '?')}")


# --------------------------------------------------------------------------------------
# functional API
# --------------------------------------------------------------------------------------

def append_kv(k, v, kv_cache, summaries, kv_indices, kv_indptr, kv_last_page_len, status=None, view=None) -> None:
    """Write one new token per sequence into the paged cache and refresh its page summary.

    k, v: [B, Hkv, D].  The page table already includes the new token
    (flashinfer.append_paged_kv_cache convention, benchmark/blocktopk_decoder.py:38-46).
    """
    _cuda(k, v, kv_cache, summaries, kv_indices, kv_indptr, kv_last_page_len, status)
    B = _batch_of(kv_indptr, view)
    if k.shape != (B, kv_cache.shape[3], kv_cache.shape[4]) or v.shape != k.shape:
        raise ValueError(f"k/v must be [B={B}, Hkv, D], got {tuple(k.shape)}")
    if k.dtype != kv_cache.dtype or v.dtype != kv_cache.dtype:
        raise TypeError("k, v and kv_cache must share a dtype")
    shp = _shape(B, kv_cache, kv_cache.shape[3])
    stride = 0
    if summaries is not None:
        if summaries.dtype != kv_cache.dtype or summaries.shape[1] != shp.num_kv_heads:
            raise ValueError("summaries must be [rows, Hkv, pages, D] in the cache dtype")
        stride = summaries.shape[2]
    vp, _keep = _view_ref(view)
    check(_lib.load().ktk_append_v(_ptr(k), _ptr(v), _ptr(kv_cache), _ptr(summaries), stride, _ptr(kv_indices),
                                   _ptr(kv_indptr), _ptr(kv_last_page_len), vp, ctypes.byref(shp), _ptr(status),
                                   _stream()))
    _launched()


def append_tokens(k, v, append_indptr, kv_cache, summaries, kv_indices, kv_indptr, kv_last_page_len, status=None,
                  view=None) -> None:
    """Append several tokens per sequence (prefill / chunked append) and refresh the touched page summaries.

    k, v: [total_tokens, Hkv, D] packed by sequence, append_indptr int32 [B+1]; the page table already
    includes the new tokens.  The multi-token form of flashinfer.append_paged_kv_cache
    (benchmark/blocktopk_decoder.py:38-46)."""
    _cuda(k, v, append_indptr, kv_cache, summaries, kv_indices, kv_indptr, kv_last_page_len, status)
    B = append_indptr.numel() - 1
    if k.dim() != 3 or k.shape[1:] != (kv_cache.shape[3], kv_cache.shape[4]) or v.shape != k.shape:
        raise ValueError("k/v must be [total_tokens, Hkv, D]")
    if k.dtype != kv_cache.dtype or v.dtype != kv_cache.dtype or append_indptr.dtype != torch.int32:
        raise TypeError("k, v and kv_cache must share a dtype; append_indptr must be int32")
    shp = _shape(B, kv_cache, kv_cache.shape[3])
    stride = 0 if summaries is None else summaries.shape[2]
    vp, _keep = _view_ref(view)
    check(_lib.load().ktk_append_tokens(_ptr(k), _ptr(v), _ptr(append_indptr), k.shape[0], _ptr(kv_cache),
                                        _ptr(summaries), stride, _ptr(kv_indices), _ptr(kv_indptr),
                                        _ptr(kv_last_page_len), vp, ctypes.byref(shp), _ptr(status), _stream()))
    _launched(1 if summaries is None else 2)


def build_summaries(kv_cache, summaries, kv_indices, kv_indptr, kv_last_page_len, status=None, view=None) -> None:
    """Recompute the mean-key summary of every page of every sequence."""
    _cuda(kv_cache, summaries, kv_indices, kv_indptr, kv_last_page_len, status)
    B = _batch_of(kv_indptr, view)
    shp = _shape(B, kv_cache, kv_cache.shape[3])
    if summaries.dtype != kv_cache.dtype or summaries.shape[1] != shp.num_kv_heads:
        raise ValueError("summaries must be [rows, Hkv, pages, D] in the cache dtype")
    vp, _keep = _view_ref(view)
    check(_lib.load().ktk_build_summaries_v(_ptr(kv_cache), _ptr(summaries), summaries.shape[2], _ptr(kv_indices),
                                            _ptr(kv_indptr), _ptr(kv_last_page_len), vp, ctypes.byref(shp),
                                            _ptr(status), _stream()))
    _launched()


def select_pages(q, summaries, kv_indices, kv_indptr, kv_last_page_len, topk: int, num_pages: int,
                 out=None, out_logical=None, out_scores=None, status=None, view=None):
    """Score every filled page against the query group and pick the top-k pages.

    q [B, Hq, D]; summaries [B, Hkv, n, D].  Returns int32 [B, Hkv, topk+1] physical page ids
    (descending score, ties to the lowest page, then the page being filled; unused tail -1).
    Replaces benchmark/blocktopk_decoder.py:216-221.
    """
    _cuda(q, summaries, kv_indices, kv_indptr, kv_last_page_len, out, out_logical, out_scores, status)
    B, Hq, Dh = q.shape
    Hkv = summaries.shape[1]
    if q.dtype != summaries.dtype:
        raise TypeError("q and summaries must share a dtype")
    if _batch_of(kv_indptr, view) != B:
        raise ValueError("batch mismatch between q and kv_indptr")
    width = topk + 1 if view is None else view.row_width(topk)
    if out is None:
        out = torch.empty(B, Hkv, width, dtype=torch.int32, device=q.device)
    elif out.shape[-1] < width:
        raise ValueError(f"select_pages: output rows must hold {width} entries")
    if out_logical is not None and out_logical.shape[-1] != out.shape[-1]:
        raise ValueError("select_pages: out_logical must have the row width of out")
    shp = Shape(B, Hkv, Hq // Hkv, Dh, PAGE_SIZE, _dtype_code(q), num_pages)
    vp, _keep = _view_ref(view)
    check(_lib.load().ktk_select_v(_ptr(q), _ptr(summaries), summaries.shape[2], _ptr(kv_indices), _ptr(kv_indptr),
                                   _ptr(kv_last_page_len), topk, vp, out.shape[-1], _ptr(out), _ptr(out_logical),
                                   _ptr(out_scores), ctypes.byref(shp), _ptr(status), _stream()))
    _launched()
    return out


def decode_num_splits(batch: int, num_kv_heads: int, group_size: int, max_entries: int, dtype=torch.bfloat16) -> int:
    shp = Shape(batch, num_kv_heads, group_size, HEAD_DIM, PAGE_SIZE,
                _lib.KTK_BF16 if dtype == torch.bfloat16 else _lib.KTK_F32, 0)
    return int(_lib.load().ktk_decode_num_splits(ctypes.byref(shp), max_entries))


def decode_workspace_bytes(batch: int, num_kv_heads: int, group_size: int, num_splits: int) -> int:
    shp = Shape(batch, num_kv_heads, group_size, HEAD_DIM, PAGE_SIZE, _lib.KTK_BF16, 0)
    return int(_lib.load().ktk_decode_workspace_bytes(ctypes.byref(shp), num_splits))


def _decode_args(q, kv_cache, max_entries, workspace, num_splits, variant=0):
    B, Hq, _ = q.shape
    shp = _shape(B, kv_cache, Hq)
    if q.dtype != kv_cache.dtype:
        raise TypeError("q and kv_cache must share a dtype")
    if num_splits == 0:
        # the fp32-FMA variant has no balanced partition: ask for the per-list policy
        num_splits = decode_num_splits(B, shp.num_kv_heads, shp.group_size, max_entries,
                                       torch.float32 if variant == VARIANT_SIMT else q.dtype)
    need = int(_lib.load().ktk_decode_workspace_bytes(ctypes.byref(shp), num_splits))
    if need and workspace is None:
        workspace = _shared_workspace(q.device, need)      # the balanced partition: a few MB whatever the batch
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        raise RuntimeError(f"decode with {num_splits} splits needs a {need}-byte workspace "
                           "(decode_workspace_bytes); pass one, or num_splits=1")
    return shp, num_splits, workspace


_WORKSPACES: dict = {}


def _shared_workspace(device, nbytes: int) -> torch.Tensor:
    """Per-device scratch for calls of the functional API that pass no workspace (kernels of one stream
    run in order, so they can share it; `DecodePlan` owns its own)."""
    ws = _WORKSPACES.get(device)
    if ws is None or ws.numel() < nbytes:
        ws = _WORKSPACES[device] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return ws


def sparse_decode(q, kv_cache, sel_pages, kv_indptr, kv_last_page_len, sm_scale: Optional[float] = None,
                  workspace=None, num_splits: int = 0, variant: int = 0, out=None, status=None, view=None,
                  topk: Optional[int] = None):
    """Attention of q [B, Hq, D] over the pages listed in sel_pages [B, Hkv, topk+1].

    Replaces mylib::decode -> flashinfer BatchDecodeWithPagedKVCacheWrapper.run
    (benchmark/blocktopk_decoder.py:176-178).
    """
    _cuda(q, kv_cache, sel_pages, kv_indptr, kv_last_page_len, workspace, out, status)
    width = sel_pages.shape[-1]
    if topk is None:
        if view is not None:
            raise ValueError("sparse_decode: pass topk together with a view")
        topk = width - 1
    shp, num_splits, workspace = _decode_args(q, kv_cache, width, workspace, num_splits, variant)
    if sel_pages.dtype != torch.int32 or sel_pages.numel() != shp.batch * shp.num_kv_heads * width:
        raise ValueError("sel_pages must be int32 [B, Hkv, row width]")
    if out is None:
        out = torch.empty_like(q)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    wsb = 0 if workspace is None else workspace.numel() * workspace.element_size()
    vp, _keep = _view_ref(view)
    check(_lib.load().ktk_sparse_decode_v(_ptr(q), _ptr(kv_cache), _ptr(sel_pages), topk, vp, width, _ptr(kv_indptr),
                                          _ptr(kv_last_page_len), sm_scale, _ptr(out), _ptr(workspace), wsb,
                                          num_splits, variant, ctypes.byref(shp), _ptr(status), _stream()))
    _launched(1 if num_splits == 1 else 2)
    return out


def dense_decode(q, kv_cache, kv_indices, kv_indptr, kv_last_page_len, max_pages_per_seq: int,
                 sm_scale: Optional[float] = None, workspace=None, num_splits: int = 0, variant: int = 0,
                 out=None, status=None, view=None):
    """Attention of q over every page of each sequence (benchmark/dense_decoder.py:168-170)."""
    _cuda(q, kv_cache, kv_indices, kv_indptr, kv_last_page_len, workspace, out, status)
    shp, num_splits, workspace = _decode_args(q, kv_cache, max_pages_per_seq, workspace, num_splits, variant)
    if out is None:
        out = torch.empty_like(q)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    wsb = 0 if workspace is None else workspace.numel() * workspace.element_size()
    vp, _keep = _view_ref(view)
    check(_lib.load().ktk_dense_decode_v(_ptr(q), _ptr(kv_cache), _ptr(kv_indices), _ptr(kv_indptr),
                                       _ptr(kv_last_page_len), vp, max_pages_per_seq, sm_scale, _ptr(out),
                                       _ptr(workspace), wsb, num_splits, variant, ctypes.byref(shp),
                                       _ptr(status), _stream()))
    _launched(1 if num_splits == 1 else 2)
    return out


def prefill_attention(q, q_indptr, max_new_tokens: int, kv_cache, kv_indices, kv_indptr, kv_last_page_len,
                      sm_scale: Optional[float] = None, variant: int = 0, out=None, status=None, view=None):
    """Causal attention of the new tokens of every sequence over the paged cache (the tokens are already in
    their pages: call append_tokens first).

    q [total_new, Hq, D] packed by sequence, q_indptr int32 [B+1]; the page table describes the state after
    the append.  Replaces flashinfer.single_prefill_with_kv_cache (litesys/attention/batch_cache.py:129-145).
    """
    _cuda(q, q_indptr, kv_cache, kv_indices, kv_indptr, kv_last_page_len, out, status)
    total, Hq, _ = q.shape
    B = q_indptr.numel() - 1
    shp = _shape(B, kv_cache, Hq)
    if q.dtype != kv_cache.dtype or q_indptr.dtype != torch.int32:
        raise TypeError("q and kv_cache must share a dtype; q_indptr must be int32")
    if out is None:
        out = torch.empty_like(q)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    need = int(_lib.load().ktk_prefill_workspace_bytes(total, shp.dtype, variant))
    if shp.dtype == _lib.KTK_BF16 and variant != VARIANT_SIMT and shp.group_size not in (1, 2, 4, 8):
        need = int(_lib.load().ktk_prefill_workspace_bytes(total, shp.dtype, VARIANT_SIMT))
    ws = _shared_workspace(q.device, need) if need else None
    vp, _keep = _view_ref(view)
    check(_lib.load().ktk_prefill_attention(_ptr(q), _ptr(q_indptr), total, int(max_new_tokens), _ptr(kv_cache),
                                            _ptr(kv_indices), _ptr(kv_indptr), _ptr(kv_last_page_len), vp, sm_scale,
                                            _ptr(out), _ptr(ws), need, variant, ctypes.byref(shp), _ptr(status),
                                            _stream()))
    _launched(2 if need else 1)
    return out


def paged_qk(q, kv_cache, kv_indices, kv_indptr, kv_last_page_len, logits, sm_scale: Optional[float] = None,
             status=None, view=None):
    """Scaled logits of q [B, Hq, D] against every key of each sequence, read through the page table, into the
    fp32 buffer logits [>= B, Hq, max_len] (qk of litesys/attention/cache_utils.py:173-190 on a paged cache)."""
    _cuda(q, kv_cache, kv_indices, kv_indptr, kv_last_page_len, logits, status)
    B, Hq, _ = q.shape
    shp = _shape(B, kv_cache, Hq)
    if logits.dtype != torch.float32 or logits.shape[0] < B or logits.shape[1] != Hq or q.dtype != kv_cache.dtype:
        raise ValueError("paged_qk: logits must be fp32 [rows >= B, Hq, max_len]; q in the cache dtype")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    vp, _keep = _view_ref(view)
    check(_lib.load().ktk_paged_qk(_ptr(q), _ptr(kv_cache), _ptr(kv_indices), _ptr(kv_indptr), _ptr(kv_last_page_len),
                                   vp, sm_scale, _ptr(logits), logits.shape[2], ctypes.byref(shp), _ptr(status),
                                   _stream()))
    _launched()
    return logits


def paged_sv(probs, batch: int, kv_cache, kv_indices, kv_indptr, kv_last_page_len, out=None, status=None, view=None):
    """sum_s probs[b, hq, s] * V[s] over a paged cache -> [B, Hq, D] in the cache dtype; rows of V whose
    probability is zero for the whole query group are skipped (sv of cache_utils.py:193-212)."""
    _cuda(probs, kv_cache, kv_indices, kv_indptr, kv_last_page_len, out, status)
    Hq = probs.shape[1]
    shp = _shape(batch, kv_cache, Hq)
    if out is None:
        out = torch.empty(batch, Hq, kv_cache.shape[4], dtype=kv_cache.dtype, device=kv_cache.device)
    vp, _keep = _view_ref(view)
    check(_lib.load().ktk_paged_sv(_ptr(kv_cache), _ptr(kv_indices), _ptr(kv_indptr), _ptr(kv_last_page_len), vp,
                                   _ptr(probs), probs.shape[2], _ptr(out), ctypes.byref(shp), _ptr(status), _stream()))
    _launched()
    return out


def token_topk_mask(logits, lengths, num_q_heads: int, num_kv_heads: int, topk: int, local: int, sink: int,
                    status=None):
    """topk_sparsity (litesys/attention/sparsity_utils.py:6-21) in place on logits [rows, Hq, max_len]."""
    _cuda(logits, lengths, status)
    check(_lib.load().ktk_token_topk_mask(_ptr(logits), _ptr(lengths), lengths.numel(), num_q_heads, num_kv_heads,
                                          logits.shape[2], topk, local, sink, _ptr(status), _stream()))
    _launched()
    return logits


def softmax_rows(logits, lengths):
    """In-place softmax over the first lengths[row] positions (cache_utils.py:216-226)."""
    _cuda(logits, lengths)
    check(_lib.load().ktk_softmax_rows(_ptr(logits), _ptr(lengths), lengths.numel(), logits.shape[1], logits.shape[2],
                                       _stream()))
    _launched()
    return logits


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last dimension (flashinfer.rmsnorm, benchmark/model_utils.py:12,23)."""
    _cuda(x, weight)
    if weight.dtype != x.dtype or weight.numel() != x.shape[-1]:
        raise ValueError("rmsnorm: weight must be [cols] in the dtype of x")
    out = torch.empty_like(x)
    cols = x.shape[-1]
    check(_lib.load().ktk_rmsnorm(_ptr(x), _ptr(weight), eps, _ptr(out), x.numel() // cols, cols, _dtype_code(x),
                                  _stream()))
    _launched()
    return out


def add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float):
    """(x + residual, rmsnorm(x + residual)) in one kernel; residual None -> (x, rmsnorm(x)).

    Replaces the residual add followed by mylib::layer_norm (benchmark/blocktopk_decoder.py:229-231)."""
    _cuda(x, residual, weight)
    cols = x.shape[-1]
    if weight.dtype != x.dtype or weight.numel() != cols or (residual is not None and residual.shape != x.shape):
        raise ValueError("add_rmsnorm: shapes / dtypes of x, residual and weight do not match")
    out_norm = torch.empty_like(x)
    out_sum = torch.empty_like(x) if residual is not None else None
    check(_lib.load().ktk_add_rmsnorm(_ptr(x), _ptr(residual), _ptr(weight), eps, _ptr(out_sum), _ptr(out_norm),
                                      x.numel() // cols, cols, _dtype_code(x), _stream()))
    _launched()
    return (out_sum if residual is not None else x), out_norm


def qkv_norm(proj: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, eps: float, num_q_heads: int, num_kv_heads: int,
             cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
             position_ids: Optional[torch.Tensor] = None):
    """Fused projection [B, (Hq + 2 Hkv) * 128] -> (q-normed q [B, Hq, 128], k-normed k [B, Hkv, 128], v).

    One launch for the split / contiguous / qk_norm sequence of benchmark/blocktopk_decoder.py:197-207.  With
    `cos`, `sin` ([max_positions, 128] tables) and `position_ids` [B], the rotary embedding of
    LiteSys/litesys/models/qwen3.py:102 is applied to q and k in the same launch."""
    _cuda(proj, wq, wk)
    B = proj.numel() // ((num_q_heads + 2 * num_kv_heads) * HEAD_DIM)
    q = torch.empty(B, num_q_heads, HEAD_DIM, dtype=proj.dtype, device=proj.device)
    k = torch.empty(B, num_kv_heads, HEAD_DIM, dtype=proj.dtype, device=proj.device)
    v = torch.empty(B, num_kv_heads, HEAD_DIM, dtype=proj.dtype, device=proj.device)
    if cos is None:
        check(_lib.load().ktk_qkv_norm(_ptr(proj), _ptr(wq), _ptr(wk), eps, _ptr(q), _ptr(k), _ptr(v), B, num_q_heads,
                                       num_kv_heads, _dtype_code(proj), _stream()))
    else:
        _cuda(cos, sin, position_ids)
        if cos.shape != sin.shape or cos.shape[-1] != HEAD_DIM or cos.dtype != proj.dtype or sin.dtype != proj.dtype \
                or not cos.is_contiguous() or not sin.is_contiguous() or position_ids.numel() != B:
            raise ValueError("qkv_norm: cos / sin [max_positions, 128] in the dtype of proj, one position per row")
        pos = position_ids.reshape(-1).to(torch.int64).contiguous()
        check(_lib.load().ktk_qkv_norm_rope(_ptr(proj), _ptr(wq), _ptr(wk), eps, _ptr(cos), _ptr(sin), _ptr(pos),
                                            cos.numel() // HEAD_DIM, _ptr(q), _ptr(k), _ptr(v), B, num_q_heads,
                                            num_kv_heads, _dtype_code(proj), _stream()))
    _launched()
    return q, k, v


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up (benchmark/blocktopk_decoder.py:235-236)."""
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("silu_mul: gate and up must match")
    if (gate.dim() == 2 and not gate.is_contiguous() and gate.stride(1) == 1 and up.stride(1) == 1
            and gate.stride(0) == up.stride(0)):
        # the two halves of one stacked gate/up GEMM output: rows a fixed stride apart
        if not (gate.is_cuda and up.is_cuda):
            raise ValueError("silu_mul: CUDA tensors")
        out = torch.empty(gate.shape, device=gate.device, dtype=gate.dtype)
        check(_lib.load().ktk_silu_mul_rows(_ptr(gate), _ptr(up), _ptr(out), gate.shape[0], gate.shape[1],
                                            gate.stride(0), _dtype_code(gate), _stream()))
        _launched()
        return out
    _cuda(gate, up)
    out = torch.empty_like(gate)
    check(_lib.load().ktk_silu_mul(_ptr(gate), _ptr(up), _ptr(out), gate.numel(), _dtype_code(gate), _stream()))
    _launched()
    return out


# --------------------------------------------------------------------------------------
# decode plans: what flashinfer keeps inside BatchDecodeWithPagedKVCacheWrapper
# --------------------------------------------------------------------------------------

class DecodePlan:
    """State `mylib::decode(q, kv_cache)` needs beyond its two tensors.

    The reference's op closes over a flashinfer wrapper holding the page-index buffers
    (benchmark/blocktopk_decoder.py:153-160, :171-178).  Here a plan is bound to its
    ``kv_cache`` tensor, so several layers (sparse and dense) coexist in one process.
    """

    def __init__(self, kv_cache, kv_indptr, kv_last_page_len, *, sel_pages=None, kv_indices=None,
                 max_pages_per_seq: int = 0, sm_scale: Optional[float] = None, variant: int = 0,
                 num_splits: int = 0, status=None):
        if (sel_pages is None) == (kv_indices is None):
            raise ValueError("a plan is either sparse (sel_pages) or dense (kv_indices)")
        self.kv_cache, self.kv_indptr, self.kv_last_page_len = kv_cache, kv_indptr, kv_last_page_len
        self.sel_pages, self.kv_indices = sel_pages, kv_indices
        self.max_pages_per_seq = max_pages_per_seq
        self.sm_scale, self.variant, self.status = sm_scale, variant, status
        self.num_splits = num_splits
        self.workspace = None

    def _ensure_workspace(self, q):
        B, Hq, _ = q.shape
        hkv = self.kv_cache.shape[3]
        entries = self.sel_pages.shape[-1] if self.sel_pages is not None else self.max_pages_per_seq
        if self.num_splits == 0:
            self.num_splits = decode_num_splits(B, hkv, Hq // hkv, entries,
                                                torch.float32 if self.variant == VARIANT_SIMT else q.dtype)
        need = decode_workspace_bytes(B, hkv, Hq // hkv, self.num_splits)
        if need and (self.workspace is None or self.workspace.numel() < need):
            self.workspace = torch.empty(need, dtype=torch.uint8, device=q.device)

    def run(self, q, kv_cache=None):
        """Attention of q under this plan; `kv_cache` (default: the plan's own) is the tensor the pages are read
        from -- like flashinfer's wrapper.run(q, kv_cache), which takes the cache as an argument."""
        self._ensure_workspace(q)
        cache = self.kv_cache if kv_cache is None else kv_cache
        if self.sel_pages is not None:
            return sparse_decode(q, cache, self.sel_pages, self.kv_indptr, self.kv_last_page_len,
                                 self.sm_scale, self.workspace, self.num_splits, self.variant, status=self.status)
        return dense_decode(q, cache, self.kv_indices, self.kv_indptr, self.kv_last_page_len,
                            self.max_pages_per_seq, self.sm_scale, self.workspace, self.num_splits, self.variant,
                            status=self.status)


_PLANS: dict[int, DecodePlan] = {}
_SUMMARIES: dict[int, torch.Tensor] = {}


_LAST_PLAN: list = [None]     # weak reference to the plan bound last


def bind_decode_plan(plan: DecodePlan) -> None:
    import weakref
    _PLANS[plan.kv_cache.data_ptr()] = plan
    _LAST_PLAN[0] = weakref.ref(plan)


def _plan_for(kv_cache: torch.Tensor) -> Optional[DecodePlan]:
    """The plan bound to this cache; for a cache nobody bound (a copy of a bound one, as torch.library.opcheck
    makes), the plan bound last if its cache has the same shape and dtype -- the reference's op likewise runs
    whatever cache it is handed through the one wrapper it closes over (benchmark/blocktopk_decoder.py:171-178)."""
    plan = _PLANS.get(kv_cache.data_ptr())
    if plan is None and _LAST_PLAN[0] is not None:
        last = _LAST_PLAN[0]()
        if last is not None and last.kv_cache.shape == kv_cache.shape and last.kv_cache.dtype == kv_cache.dtype \
                and last.kv_cache.device == kv_cache.device:
            plan = last
    return plan


def bind_summaries(kv_cache: torch.Tensor, summaries: Optional[torch.Tensor]) -> None:
    """Make `mylib::update_kv` on this cache also maintain `summaries`."""
    if summaries is None:
        _SUMMARIES.pop(kv_cache.data_ptr(), None)
    else:
        _SUMMARIES[kv_cache.data_ptr()] = summaries


def unbind(kv_cache: torch.Tensor) -> None:
    unbind_address(kv_cache.data_ptr())


def unbind_address(address: int) -> None:
    """Forget the plan and summaries bound to the cache at `address` (a layer that is deleted calls this, so
    that a later cache which happens to get the same address does not inherit them)."""
    _PLANS.pop(address, None)
    _SUMMARIES.pop(address, None)


# --------------------------------------------------------------------------------------
# torch custom ops (reference names and schemas)
# --------------------------------------------------------------------------------------

torch.library.define(
    "mylib::update_kv",
    "(Tensor k, Tensor v, Tensor kv_append_indptr, Tensor(a!) kv_cache, Tensor kv_page_indices, "
    "Tensor kv_page_indptr, Tensor cachelen) -> ()",
)


@torch.library.impl("mylib::update_kv", "cuda")
def _update_kv(k, v, kv_append_indptr, kv_cache, kv_page_indices, kv_page_indptr, kv_page_last_len):
    summ = _SUMMARIES.get(kv_cache.data_ptr())
    if k.shape[0] == kv_page_indptr.numel() - 1:
        # one token per sequence (decode): kv_append_indptr is arange(B+1) and need not be read
        append_kv(k, v, kv_cache, summ, kv_page_indices, kv_page_indptr, kv_page_last_len)
    else:
        append_tokens(k, v, kv_append_indptr, kv_cache, summ, kv_page_indices, kv_page_indptr, kv_page_last_len)


@torch.library.register_fake("mylib::update_kv")
def _update_kv_fake(k, v, kv_append_indptr, kv_cache, kv_page_indices, kv_page_indptr, kv_page_last_len):
    return None


torch.library.define("mylib::decode", "(Tensor q, Tensor kv_cache) -> Tensor")


@torch.library.impl("mylib::decode", "cuda")
def _decode(q, kv_cache):
    plan = _plan_for(kv_cache)
    if plan is None:
        raise RuntimeError("mylib::decode: no DecodePlan bound to this kv_cache (bind_decode_plan)")
    return plan.run(q, kv_cache)


@torch.library.register_fake("mylib::decode")
def _decode_fake(q, kv_cache):
    return torch.empty_like(q)


torch.library.define("mylib::qk_norm", "(Tensor q, float variance_epsilon, Tensor weight) -> Tensor")


@torch.library.impl("mylib::qk_norm", "cuda")
def _qk_norm(q, variance_epsilon, weight):
    return rmsnorm(q.contiguous(), weight, variance_epsilon)


@torch.library.register_fake("mylib::qk_norm")
def _qk_norm_fake(q, variance_epsilon, weight):
    return torch.empty_like(q)


torch.library.define("mylib::layer_norm", "(Tensor input, float variance_epsilon, Tensor weight) -> Tensor")


@torch.library.impl("mylib::layer_norm", "cuda")
def _layer_norm(input, variance_epsilon, weight):
    return rmsnorm(input.contiguous(), weight, variance_epsilon)


@torch.library.register_fake("mylib::layer_norm")
def _layer_norm_fake(input, variance_epsilon, weight):
    return torch.empty_like(input)


torch.library.define(
    "ktk::select_pages",
    "(Tensor q, Tensor summaries, Tensor kv_indices, Tensor kv_indptr, Tensor kv_last_page_len, int topk, "
    "int num_pages) -> Tensor",
)


@torch.library.impl("ktk::select_pages", "cuda")
def _select_pages(q, summaries, kv_indices, kv_indptr, kv_last_page_len, topk, num_pages):
    return select_pages(q, summaries, kv_indices, kv_indptr, kv_last_page_len, topk, num_pages)


@torch.library.register_fake("ktk::select_pages")
def _select_pages_fake(q, summaries, kv_indices, kv_indptr, kv_last_page_len, topk, num_pages):
    return torch.empty(q.shape[0], summaries.shape[1], topk + 1, dtype=torch.int32, device=q.device)


torch.library.define(
    "ktk::sparse_decode",
    "(Tensor q, Tensor kv_cache, Tensor sel_pages, Tensor kv_indptr, Tensor kv_last_page_len) -> Tensor",
)


@torch.library.impl("ktk::sparse_decode", "cuda")
def _sparse_decode(q, kv_cache, sel_pages, kv_indptr, kv_last_page_len):
    return sparse_decode(q, kv_cache, sel_pages, kv_indptr, kv_last_page_len, num_splits=1)


@torch.library.register_fake("ktk::sparse_decode")
def _sparse_decode_fake(q, kv_cache, sel_pages, kv_indptr, kv_last_page_len):
    return torch.empty_like(q)


torch.library.define(
    "ktk::dense_decode",
    "(Tensor q, Tensor kv_cache, Tensor kv_indices, Tensor kv_indptr, Tensor kv_last_page_len) -> Tensor",
)


@torch.library.impl("ktk::dense_decode", "cuda")
def _dense_decode(q, kv_cache, kv_indices, kv_indptr, kv_last_page_len):
    return dense_decode(q, kv_cache, kv_indices, kv_indptr, kv_last_page_len, 1, num_splits=1)


@torch.library.register_fake("ktk::dense_decode")
def _dense_decode_fake(q, kv_cache, kv_indices, kv_indptr, kv_last_page_len):
    return torch.empty_like(q)


torch.library.define(
    "ktk::append_kv_with_summary",
    "(Tensor k, Tensor v, Tensor(a!) kv_cache, Tensor(b!) summaries, Tensor kv_indices, Tensor kv_indptr, "
    "Tensor kv_last_page_len) -> ()",
)


@torch.library.impl("ktk::append_kv_with_summary", "cuda")
def _append_kv_with_summary(k, v, kv_cache, summaries, kv_indices, kv_indptr, kv_last_page_len):
    append_kv(k, v, kv_cache, summaries, kv_indices, kv_indptr, kv_last_page_len)


@torch.library.register_fake("ktk::append_kv_with_summary")
def _append_kv_with_summary_fake(k, v, kv_cache, summaries, kv_indices, kv_indptr, kv_last_page_len):
    return None


# --------------------------------------------------------------------------------------
# the fused glue kernels and the selection as torch ops, so that torch.compile(fullgraph=True)
# traces a layer forward end to end the way it traces the reference's
# (benchmark/blocktopk.py:41-43); the functional wrappers above stay the eager entry points
# --------------------------------------------------------------------------------------

torch.library.define("ktk::rms_norm", "(Tensor x, Tensor weight, float eps) -> Tensor")


@torch.library.impl("ktk::rms_norm", "cuda")
def _rms_norm_op(x, weight, eps):
    return add_rmsnorm(x, None, weight, eps)[1]


@torch.library.register_fake("ktk::rms_norm")
def _rms_norm_fake(x, weight, eps):
    return torch.empty_like(x)


torch.library.define("ktk::add_rms_norm", "(Tensor x, Tensor residual, Tensor weight, float eps) -> (Tensor, Tensor)")


@torch.library.impl("ktk::add_rms_norm", "cuda")
def _add_rms_norm_op(x, residual, weight, eps):
    return add_rmsnorm(x, residual, weight, eps)


@torch.library.register_fake("ktk::add_rms_norm")
def _add_rms_norm_fake(x, residual, weight, eps):
    return torch.empty_like(x), torch.empty_like(x)


torch.library.define(
    "ktk::qkv_norm",
    "(Tensor proj, Tensor wq, Tensor wk, float eps, int num_q_heads, int num_kv_heads) -> (Tensor, Tensor, Tensor)")


@torch.library.impl("ktk::qkv_norm", "cuda")
def _qkv_norm_op(proj, wq, wk, eps, num_q_heads, num_kv_heads):
    return qkv_norm(proj, wq, wk, eps, num_q_heads, num_kv_heads)


@torch.library.register_fake("ktk::qkv_norm")
def _qkv_norm_fake(proj, wq, wk, eps, num_q_heads, num_kv_heads):
    B = proj.numel() // ((num_q_heads + 2 * num_kv_heads) * HEAD_DIM)
    return (proj.new_empty(B, num_q_heads, HEAD_DIM), proj.new_empty(B, num_kv_heads, HEAD_DIM),
            proj.new_empty(B, num_kv_heads, HEAD_DIM))


torch.library.define("ktk::silu_mul", "(Tensor gate, Tensor up) -> Tensor")


@torch.library.impl("ktk::silu_mul", "cuda")
def _silu_mul_op(gate, up):
    return silu_mul(gate, up)


@torch.library.register_fake("ktk::silu_mul")
def _silu_mul_fake(gate, up):
    return torch.empty_like(gate)


torch.library.define(
    "ktk::select_pages_into",
    "(Tensor q, Tensor summaries, Tensor kv_indices, Tensor kv_indptr, Tensor kv_last_page_len, int topk, "
    "int num_pages, Tensor(a!) out, Tensor(b!) status) -> ()",
)


@torch.library.impl("ktk::select_pages_into", "cuda")
def _select_pages_into(q, summaries, kv_indices, kv_indptr, kv_last_page_len, topk, num_pages, out, status):
    select_pages(q, summaries, kv_indices, kv_indptr, kv_last_page_len, topk, num_pages, out=out, status=status)


@torch.library.register_fake("ktk::select_pages_into")
def _select_pages_into_fake(q, summaries, kv_indices, kv_indptr, kv_last_page_len, topk, num_pages, out, status):
    return None
