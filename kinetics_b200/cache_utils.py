"""The functions of ``LiteSys/litesys/attention/cache_utils.py`` and the block top-k branch of
``sparsity_utils.attn_logits_processor`` (plus its token top-k branch), with the reference's names, arguments and in-place
behaviour, on CUDA kernels of ``libktk.so`` (``csrc/ktk_dense_chain.cu``).

They keep the reference's own data layout -- unpaged ``[max_batch, Hkv, max_len, D]`` caches and an
fp32 ``[rows, Hq, max_len]`` logits buffer -- so that the reference's ``BatchKVManager.decode``
(``batch_cache.py:154-168``) runs on them line for line.  They read every key and value of a
sequence; ``kinetics_b200.BatchKVManager`` gets the same result from the selected pages only and is
the fast path.  As in the reference, ``offset`` is indexed by the ROW of the active batch and the
cache slot is ``batch_idx[row]`` (``cache_utils.py:67,106,149``).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, ops
from ._lib import check
from .batch_cache import preprocess_sparse_args  # noqa: F401  (same module surface as sparsity_utils.py)

_STATUS: dict = {}


def _status(device) -> torch.Tensor:
    st = _STATUS.get(device)
    if st is None:
        st = _STATUS[device] = ops.new_status(device)
    return st


def check_status(device) -> None:
    """Raise if one of the functions met a slot or position outside its cache."""
    ops.raise_on_status(_status(torch.device(device)))


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.KTK_BF16
    if t.dtype == torch.float32:
        return _lib.KTK_F32
    raise TypeError(f"{t.dtype}: only bfloat16 and float32 are built")


def _cuda(*ts):
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("kinetics_b200.cache_utils: CUDA tensors only, there is no CPU fallback")


def _i64(t):
    return t if t.dtype == torch.int64 and t.is_contiguous() else t.to(torch.int64).contiguous()


def _i32(t):
    return t if t.dtype == torch.int32 and t.is_contiguous() else t.to(torch.int32).contiguous()


def copy_to_cache(key_cache, key, batch_id, offset):
    """cache_utils.py:40-51: ``key`` [B, Hkv, 1, D] -> ``key_cache[batch_id[b], h, offset[b], :]``."""
    _cuda(key_cache, key, batch_id, offset)
    B, H, _, D = key.shape
    if key.stride(3) != 1 or not key_cache.is_contiguous() or key.dtype != key_cache.dtype:
        raise ValueError("copy_to_cache: contiguous cache, unit stride along head_dim, one dtype")
    check(_lib.load().ktk_copy_to_cache(_p(key_cache), _p(key), _p(_i64(batch_id)), _p(_i32(offset)), B, H,
                                        key_cache.shape[0], key_cache.shape[2], D, key.stride(0), key.stride(1),
                                        _dt(key), _p(_status(key.device)), _stream()))


def qk(query, key, batch_idx, offset, logits_buffer, BLOCK_SEQ):
    """cache_utils.py:173-190: scaled logits of ``query`` [B, Hq, 1, D] against ``key`` (the key cache) into
    ``logits_buffer`` [rows, Hq, max_len] fp32, -inf behind ``offset[b]`` inside the blocks it touches."""
    _cuda(query, key, batch_idx, offset, logits_buffer)
    B, Hq, _, D = query.shape
    _, Hkv, max_len, _ = key.shape
    if logits_buffer.dtype != torch.float32 or logits_buffer.shape[1] != Hq or logits_buffer.shape[2] != max_len \
            or not logits_buffer.is_contiguous() or not key.is_contiguous():
        raise ValueError("qk: logits_buffer must be contiguous fp32 [rows, Hq, max_len]")
    q = query.reshape(B, Hq, D).contiguous()
    check(_lib.load().ktk_qk(_p(q), _p(key), _p(_i64(batch_idx)), _p(_i32(offset)), _p(logits_buffer), B, Hq, Hkv,
                             key.shape[0], max_len, D, BLOCK_SEQ, _dt(key), _p(_status(key.device)), _stream()))


def softmax(logits_buffer, batch_idx, offset):
    """cache_utils.py:216-226: in place over the first ``offset[b]`` positions of the first len(batch_idx) rows."""
    _cuda(logits_buffer, offset)
    check(_lib.load().ktk_softmax_rows(_p(logits_buffer), _p(_i32(offset)), len(batch_idx), logits_buffer.shape[1],
                                       logits_buffer.shape[2], _stream()))


def sv(value, batch_idx, offset, logits_buffer, output_buffer, BLOCK_SEQ):
    """cache_utils.py:193-212: probabilities x values -> [B, Hq, D] in the cache dtype.  ``output_buffer`` (the
    reference's per-block partials) is accepted for the signature's sake and left untouched."""
    _cuda(value, batch_idx, offset, logits_buffer)
    B = len(batch_idx)
    Hq = logits_buffer.shape[1]
    _, Hkv, max_len, D = value.shape
    out = torch.empty(B, Hq, D, dtype=value.dtype, device=value.device)
    check(_lib.load().ktk_sv(_p(value), _p(_i64(batch_idx)), _p(_i32(offset)), _p(logits_buffer), _p(out), B, Hq, Hkv,
                             value.shape[0], max_len, D, _dt(value), _p(_status(value.device)), _stream()))
    return out


def blockwise_topk_sparsity(logits_triton, offset, num_query_heads, num_key_value_heads, topk_block, local, sink=4,
                            block_size=16):
    """sparsity_utils.py:24-47, for every row of the buffer, without the per-row host loop."""
    if block_size != ops.PAGE_SIZE:
        raise NotImplementedError(f"block_size must be {ops.PAGE_SIZE}")
    _cuda(logits_triton, offset)
    rows = min(logits_triton.shape[0], offset.numel())
    check(_lib.load().ktk_block_topk_mask(_p(logits_triton), _p(_i32(offset)), rows, num_query_heads,
                                          num_key_value_heads, logits_triton.shape[2], topk_block, local, sink,
                                          _p(_status(logits_triton.device)), _stream()))
    return logits_triton


def topk_sparsity(logits_triton, offset, num_query_heads, num_key_value_heads, topk, local, sink=4):
    """sparsity_utils.py:6-21, for every row of the buffer, without the per-row host loop: rows longer than
    sink + topk + local keep the sink, the `local` newest tokens and the topk tokens in between with the
    largest group-mean logit."""
    _cuda(logits_triton, offset)
    rows = min(logits_triton.shape[0], offset.numel())
    check(_lib.load().ktk_token_topk_mask(_p(logits_triton), _p(_i32(offset)), rows, num_query_heads,
                                          num_key_value_heads, logits_triton.shape[2], topk, local, sink,
                                          _p(_status(logits_triton.device)), _stream()))
    return logits_triton


def attn_logits_processor(logits_triton, offset, num_query_heads, num_key_value_heads, layer_idx, **kwargs):
    """sparsity_utils.py:217-249.  The block top-k mask, the token top-k mask and "no sparsity" are built; the
    other masks raise."""
    if (not kwargs["use_sparsity"]) or (layer_idx in kwargs["attn_layer_skip"]):
        return logits_triton
    if kwargs.get("attn_topk") is not None:
        return topk_sparsity(logits_triton, offset, num_query_heads, num_key_value_heads, kwargs["attn_topk"],
                             kwargs["attn_local"])
    if kwargs.get("attn_block_topk") is None or kwargs.get("attn_stride") is not None:
        raise NotImplementedError("only attn_block_topk and attn_topk (+ attn_local) are built; strided, random and "
                                  "local-only masks are not")
    return blockwise_topk_sparsity(logits_triton, offset, num_query_heads, num_key_value_heads,
                                   kwargs["attn_block_topk"], kwargs["attn_local"],
                                   block_size=kwargs.get("attn_block_size", 16))
