"""CPU oracle for block top-k paged decode attention -- TEST INFRASTRUCTURE ONLY.

Python face of ``ktk_oracle.c`` (ctypes) plus a torch restatement of the reference's own
PyTorch lines.  Only the test-suite, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this module; the product (``kinetics_b200``) never does.

Two layers:

* ``summaries / scores / select / decode / append`` -- the *defining* restatement
  (``ktk_oracle.c``): fixed fp32 summation order for scores, ties to the lowest page,
  float64 attention.  The CUDA kernels are compared with these.
* ``reference_torch_*`` -- the reference's PyTorch statements on CPU tensors, kept as close
  to the original lines as a paged layout allows (``benchmark/blocktopk_decoder.py:216-221``
  for the selection, gather + ``softmax(q K^T / sqrt(D)) V`` for the attention that the
  reference delegates to flashinfer at ``:176-178``).  This is what the benchmark times as
  "the reference's CPU path".

Layouts are those of ``include/ktk.h``.  Tensors are CPU torch tensors (fp32 or bf16).
"""
from __future__ import annotations

import ctypes
import math
import subprocess
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB = None

D = 128
P = 16


def build(force: bool = False) -> Path:
    """Compile ``ktk_oracle.c`` (gcc, see Makefile)."""
    so = _HERE / "libktk_oracle.so"
    if force or not so.exists() or so.stat().st_mtime < (_HERE / "ktk_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True)
    return so


def _lib():
    global _LIB
    if _LIB is None:
        so = _HERE / "libktk_oracle.so"
        if not so.exists():
            build()
        _LIB = ctypes.CDLL(str(so))
    return _LIB


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"oracle: dtype {t.dtype} not supported")


def _p(t):
    if t is None:
        return ctypes.c_void_p(0)
    assert t.device.type == "cpu" and t.is_contiguous()
    return ctypes.c_void_p(t.data_ptr())


def _i32(t):
    assert t.dtype == torch.int32
    return _p(t)


def summaries(kv_cache, kv_indices, kv_indptr, kv_last_page_len, summary_stride: int):
    """Mean key of every page -> [B, Hkv, summary_stride, D] (unused rows zero)."""
    B = kv_indptr.numel() - 1
    Hkv = kv_cache.shape[3]
    out = torch.zeros(B, Hkv, summary_stride, D, dtype=kv_cache.dtype)
    _lib().ktko_summaries(_p(kv_cache), _p(out), ctypes.c_int64(summary_stride), _i32(kv_indices),
                          _i32(kv_indptr), _i32(kv_last_page_len), B, Hkv, _dt(kv_cache))
    return out


def append(k, v, kv_cache, summ, kv_indices, kv_indptr, kv_last_page_len):
    """In-place append of one token per sequence (page table already advanced)."""
    B, Hkv = k.shape[0], k.shape[1]
    stride = summ.shape[2] if summ is not None else 0
    _lib().ktko_append(_p(k), _p(v), _p(kv_cache), _p(summ), ctypes.c_int64(stride), _i32(kv_indices),
                       _i32(kv_indptr), _i32(kv_last_page_len), B, Hkv, _dt(k))


def append_tokens(k, v, append_indptr, kv_cache, kv_indices, kv_indptr, kv_last_page_len, sink: int = 0):
    """In-place append of several tokens per sequence (k, v [total, Hkv, D] packed by sequence)."""
    B = append_indptr.numel() - 1
    _lib().ktko_append_tokens(_p(k), _p(v), _i32(append_indptr), _p(kv_cache), _i32(kv_indices), _i32(kv_indptr),
                              _i32(kv_last_page_len), sink, B, kv_cache.shape[3], _dt(k))


def scores(q, summ, kv_indptr):
    """fp32 page scores in the contract's summation order -> [B, Hkv, summary_stride]."""
    B, Hq = q.shape[0], q.shape[1]
    Hkv, stride = summ.shape[1], summ.shape[2]
    G = Hq // Hkv
    out = torch.full((B, Hkv, stride), float("nan"), dtype=torch.float32)
    _lib().ktko_scores(_p(q), _p(summ), ctypes.c_int64(stride), _i32(kv_indptr), _p(out), B, Hkv, G, _dt(q))
    return out


def select_from_scores(sc, kv_indices, kv_indptr, topk: int):
    """(physical, logical) int32 [B, Hkv, topk+1]; descending score, ties to the lowest page."""
    B, Hkv, stride = sc.shape
    phys = torch.empty(B, Hkv, topk + 1, dtype=torch.int32)
    logical = torch.empty(B, Hkv, topk + 1, dtype=torch.int32)
    _lib().ktko_select(_p(sc), ctypes.c_int64(stride), _i32(kv_indices), _i32(kv_indptr), topk,
                       _p(phys), _p(logical), B, Hkv)
    return phys, logical


def select(q, summ, kv_indices, kv_indptr, topk: int):
    return select_from_scores(scores(q, summ, kv_indptr), kv_indices, kv_indptr, topk)


def decode(q, kv_cache, entries, topk: int, kv_indptr, kv_last_page_len, sm_scale: float):
    """float64 attention over the listed pages -> fp32 [B, Hq, D].  topk < 0: dense (entries = kv_indices)."""
    B, Hq = q.shape[0], q.shape[1]
    Hkv = kv_cache.shape[3]
    out = torch.empty(B, Hq, D, dtype=torch.float32)
    _lib().ktko_decode(_p(q), _p(kv_cache), _i32(entries), topk, _i32(kv_indptr), _i32(kv_last_page_len),
                       ctypes.c_float(sm_scale), _p(out), B, Hkv, Hq // Hkv, _dt(q))
    return out


# --------------------------------------------------------------------------------------
# The same under a page view (sink_tokens, local_tokens): LiteSys semantics
# --------------------------------------------------------------------------------------

def back_max(local: int) -> int:
    return 1 if local <= 1 else 1 + (local - 1 + P - 1) // P


def row_width(topk: int, sink: int, local: int) -> int:
    return (1 if sink > 0 else 0) + topk + back_max(local)


def summaries_v(kv_cache, kv_indices, kv_indptr, kv_last_page_len, summary_stride: int, sink: int):
    B = kv_indptr.numel() - 1
    Hkv = kv_cache.shape[3]
    out = torch.zeros(B, Hkv, summary_stride, D, dtype=kv_cache.dtype)
    _lib().ktko_summaries_v(_p(kv_cache), _p(out), ctypes.c_int64(summary_stride), _i32(kv_indices),
                            _i32(kv_indptr), _i32(kv_last_page_len), sink, B, Hkv, _dt(kv_cache))
    return out


def select_v(q, summ, kv_indices, kv_indptr, kv_last_page_len, topk: int, sink: int, local: int):
    """(physical, logical, scores) under the view; rows are row_width(topk, sink, local) wide."""
    B, Hq = q.shape[0], q.shape[1]
    Hkv, stride = summ.shape[1], summ.shape[2]
    sc = torch.full((B, Hkv, stride), float("nan"), dtype=torch.float32)
    _lib().ktko_scores_v(_p(q), _p(summ), ctypes.c_int64(stride), _i32(kv_indptr), _i32(kv_last_page_len), sink,
                         local, _p(sc), B, Hkv, Hq // Hkv, _dt(q))
    w = row_width(topk, sink, local)
    phys = torch.empty(B, Hkv, w, dtype=torch.int32)
    logical = torch.empty(B, Hkv, w, dtype=torch.int32)
    _lib().ktko_select_v(_p(sc), ctypes.c_int64(stride), _i32(kv_indices), _i32(kv_indptr), _i32(kv_last_page_len),
                         topk, sink, local, w, _p(phys), _p(logical), B, Hkv)
    return phys, logical, sc


def decode_v(q, kv_cache, entries, topk: int, kv_indptr, kv_last_page_len, sm_scale: float, sink: int, local: int):
    B, Hq = q.shape[0], q.shape[1]
    Hkv = kv_cache.shape[3]
    out = torch.empty(B, Hq, D, dtype=torch.float32)
    w = entries.shape[-1] if topk >= 0 else 0
    _lib().ktko_decode_v(_p(q), _p(kv_cache), _i32(entries), topk, sink, local, w, _i32(kv_indptr),
                         _i32(kv_last_page_len), ctypes.c_float(sm_scale), _p(out), B, Hkv, Hq // Hkv, _dt(q))
    return out


# --------------------------------------------------------------------------------------
# The reference's own PyTorch statements, on CPU tensors
# --------------------------------------------------------------------------------------

def reference_torch_select(q, compressed_key_cache, page_table, topk: int):
    """benchmark/blocktopk_decoder.py:216-221 for a uniform batch with one kv head.

    q [B, G, D]; compressed_key_cache [B, n, D]; page_table [B, n+1] physical ids.
    Returns int32 [B, topk+1].  The reference indexes its flat table as
    ``paged_kv_indices[idx * B + b]``, which addresses a [B, n+1]-major table with an
    [n+1, B]-major index; the intended gather ``page_table[b, idx]`` is used here.
    """
    csim = torch.einsum("b g d, b n d -> b g n", q, compressed_key_cache).mean(dim=1)
    idx = torch.topk(csim, topk, dim=-1).indices
    phys = torch.gather(page_table[:, :-1], 1, idx)
    phys = torch.cat([phys, page_table[:, -1:]], dim=-1)
    return phys.to(torch.int32).contiguous()


def reference_torch_decode(q, kv_cache, sel_pages, last_page_len: int, sm_scale: float):
    """Attention over the listed pages in plain torch (uniform batch, one kv head).

    q [B, G, D]; kv_cache [pages, 2, P, 1, D]; sel_pages [B, k+1]; every listed page full except
    the last, which holds ``last_page_len`` tokens.  Same math as the reference's
    ``softmax(logits) @ V`` (LiteSys cache_utils.py:86,116-130,165), restricted to the pages.
    """
    B, G, _ = q.shape
    kv = kv_cache[sel_pages.long()]                   # [B, k+1, 2, P, 1, D]
    k = kv[:, :, 0, :, 0, :].reshape(B, -1, D)
    v = kv[:, :, 1, :, 0, :].reshape(B, -1, D)
    ntok = (sel_pages.shape[1] - 1) * P + last_page_len
    k, v = k[:, :ntok], v[:, :ntok]
    logits = torch.einsum("b g d, b s d -> b g s", q.float(), k.float()) * sm_scale
    p = torch.softmax(logits, dim=-1)
    return torch.einsum("b g s, b s d -> b g d", p, v.float())


def token_topk_decode(q, k, v, lens, topk: int, local: int, sink: int, sm_scale: float):
    """Token-level top-k attention on contiguous histories -- the restatement of the reference chain
    qk -> topk_sparsity -> softmax -> sv (LiteSys/litesys/attention/sparsity_utils.py:6-21,
    cache_utils.py:54-226) in plain torch, fp32 logits as in the reference, float64 softmax and sum.

    q [B, Hq, D]; k, v [B, Hkv, L, D]; lens[b] tokens of sequence b.  Rows longer than sink + topk + local keep
    the sink, the `local` newest tokens and the topk tokens in between with the largest logit averaged over the
    query group (a stable descending sort: ties to the lower position).
    Returns (out [B, Hq, D] fp32, kept [B, Hkv, topk] int32 ascending positions or -1)."""
    B, Hq, Dh = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    out = torch.zeros(B, Hq, Dh, dtype=torch.float32)
    kept = torch.full((B, Hkv, topk), -1, dtype=torch.int32)
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            continue
        for h in range(Hkv):
            qg = q[b, h * G:(h + 1) * G].float()
            logits = (qg @ k[b, h, :n].float().t()) * sm_scale                   # [G, n] fp32
            mask = torch.ones(n, dtype=torch.bool)
            if n > sink + topk + local:
                mean = logits[:, sink:n - local].sum(0) / G
                order = torch.sort(-(mean + 0.0), stable=True).indices[:topk]
                mask[sink:n - local] = False
                mask[sink + order] = True
                kept[b, h] = (sink + torch.sort(order).values).to(torch.int32)
            lg = logits.double().masked_fill(~mask[None], float("-inf"))
            out[b, h * G:(h + 1) * G] = (torch.softmax(lg, dim=-1) @ v[b, h, :n].double()).float()
    return out, kept


def default_scale() -> float:
    return 1.0 / math.sqrt(D)
