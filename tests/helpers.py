"""Shared builders for the tests: paged state from contiguous histories, golden loading."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from golden.cases import CASES, LITESYS_CASES, LITESYS_TOKEN_CASES, SINK, D, P, make_case  # noqa: F401

GOLDEN = Path(__file__).resolve().parent / "golden"


def torch_dtype(name: str):
    return torch.bfloat16 if name == "bfloat16" else torch.float32


def paged_state(k, v, lens, dtype, seed=0, extra_pages=7, summary_stride=None, fill=None, sink=0):
    """Scatter contiguous histories k, v [B, Hkv, L, D] (fp32 numpy/torch) into a paged cache.

    Returns dict(kv_cache [N,2,P,Hkv,D], kv_indices, kv_indptr, kv_last_page_len, page_table list,
    num_pages, summary_stride).  Physical pages are a seeded random permutation; unused slots of
    the cache hold `fill` (default: NaN, so that a kernel reading past a fill level is caught).
    """
    k = torch.as_tensor(k)
    v = torch.as_tensor(v)
    lens = [int(x) for x in lens]
    B, Hkv = k.shape[0], k.shape[1]
    # with a sink, logical page 0 holds tokens [0, sink) and page p >= 1 tokens [sink + 16(p-1), sink + 16p)
    def n_pages_of(n):
        if sink == 0:
            return (n + P - 1) // P
        return 0 if n == 0 else (1 if n <= sink else 1 + (n - sink + P - 1) // P)

    def span(p, n):
        if sink == 0:
            return p * P, min(n, (p + 1) * P)
        if p == 0:
            return 0, min(n, sink)
        return sink + (p - 1) * P, min(n, sink + p * P)

    npages = [n_pages_of(n) for n in lens]
    total = sum(npages) + extra_pages
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(total, generator=g).tolist()
    cache = torch.full((total, 2, P, Hkv, D), float("nan") if fill is None else fill, dtype=torch.float32)
    indices, indptr, last = [], [0], []
    cur = 0
    for b in range(B):
        pages = perm[cur:cur + npages[b]]
        cur += npages[b]
        indices += pages
        indptr.append(len(indices))
        last.append(lens[b] - span(npages[b] - 1, lens[b])[0] if npages[b] else 0)
        for p, phys in enumerate(pages):
            t0, t1 = span(p, lens[b])
            cache[phys, 0, : t1 - t0] = k[b, :, t0:t1].permute(1, 0, 2)
            cache[phys, 1, : t1 - t0] = v[b, :, t0:t1].permute(1, 0, 2)
    if summary_stride is None:
        summary_stride = max(npages + [1]) + 3
    return dict(
        kv_cache=cache.to(dtype).contiguous(),
        kv_indices=torch.tensor(indices + [0], dtype=torch.int32)[: max(len(indices), 1)].contiguous(),
        kv_indptr=torch.tensor(indptr, dtype=torch.int32),
        kv_last_page_len=torch.tensor(last, dtype=torch.int32),
        num_pages=total, summary_stride=summary_stride, npages=npages,
    )


def case_state(name: str, seed=0):
    """Golden case -> (case dict, paged state, q tensor in the case dtype)."""
    case = make_case(name)
    dt = torch_dtype(case["dtype"])
    st = paged_state(case["k"], case["v"], case["lens"], dt, seed=seed, sink=case["sink"])
    q = torch.from_numpy(case["q"]).to(dt)
    return case, st, q


def load_golden(name: str):
    z = np.load(GOLDEN / f"{name}.npz")
    return {k: z[k] for k in z.files}


def random_case(seed, B, Hkv, G, lens, dtype, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    L = max(max(lens), 1)
    q = torch.randn(B, Hkv * G, D, generator=g) * scale
    k = torch.randn(B, Hkv, L, D, generator=g) * scale
    v = torch.randn(B, Hkv, L, D, generator=g)
    if dtype == torch.bfloat16:
        q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    return q.to(dtype), k, v


def to_dev(st: dict, device):
    return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in st.items()}
