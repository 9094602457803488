"""Deterministic inputs of the golden cases (shared by make_golden.py and the tests).

Each case is a batch of contiguous per-sequence K/V histories plus the decode-step query;
the tests scatter them into a paged cache through a seeded page table.  Values come from
numpy's PCG64 stream; ``checksum`` guards against a drifting generator.
"""
from __future__ import annotations

import hashlib

import numpy as np

D = 128
P = 16

# name: (seed, Hkv, G, lens, topk, dtype)   lens count the token the step appends
# The bf16 seeds were picked so that the k-th and (k+1)-th block scores differ by more than 2 %
# of the score spread: a bf16 page summary carries ~0.4 % rounding noise that the reference's
# fp32 block mean does not, and a closer call could legitimately go either way.
CASES = {
    # the CPU-runnable reference case: B=4, 1 kv head, GQA 4, 2048-token context (+ the new token), top-k 16, fp32
    "cfg1_fp32": (1234, 1, 4, [2049, 2049, 2049, 2049], 16, "float32"),
    "ragged_bf16": (2591, 2, 4, [33, 300, 273, 1029, 640], 8, "bfloat16"),
    "ragged_fp32": (1302, 2, 2, [129, 400, 97], 4, "float32"),
    "group8_bf16": (1413, 1, 8, [700, 528], 12, "bfloat16"),
    "group1_bf16": (1544, 4, 1, [260, 513], 6, "bfloat16"),
    # at or below the budget: nothing is dropped (81 tokens is the first length that selects)
    "short_fp32": (1305, 2, 2, [1, 16, 40, 80, 81], 4, "float32"),
}


# LiteSys semantics (sink of 4 tokens, `local` newest tokens always kept, 16-token blocks counted from
# the end of the sink): name -> (seed, Hkv, G, lens, topk, local, dtype)
SINK = 4
LITESYS_CASES = {
    "ls_fp32_local0": (2101, 2, 2, [100, 260, 53, 4, 3, 21, 68, 84], 4, 0, "float32"),
    "ls_bf16_local7": (2392, 2, 4, [300, 1029, 77], 8, 7, "bfloat16"),
    "ls_bf16_local64": (2113, 1, 4, [700, 400], 6, 64, "bfloat16"),
}


# Token-level top-k (`attn_topk`, sparsity_utils.py:6-21), same layout: name -> (seed, Hkv, G, lens, topk, local, dtype).
# Lengths at and around sink + topk + local (the first length that selects is one more than that).
LITESYS_TOKEN_CASES = {
    "ls_tok_fp32": (3101, 2, 2, [300, 45, 44, 7, 130, 46], 32, 8, "float32"),
    "ls_tok_bf16": (3201, 1, 4, [700, 1029, 90], 64, 16, "bfloat16"),
}


def _bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16-representable fp32 (ties to even)."""
    u = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def make_case(name: str) -> dict:
    local = None
    if name in LITESYS_TOKEN_CASES:
        seed, hkv, g, lens, topk, local, dtype = LITESYS_TOKEN_CASES[name]
    elif name in LITESYS_CASES:
        seed, hkv, g, lens, topk, local, dtype = LITESYS_CASES[name]
    else:
        seed, hkv, g, lens, topk, dtype = CASES[name]
    rng = np.random.default_rng(seed)
    B, L = len(lens), max(lens)
    q = rng.standard_normal((B, hkv * g, D), dtype=np.float32)
    k = rng.standard_normal((B, hkv, L, D), dtype=np.float32)
    v = rng.standard_normal((B, hkv, L, D), dtype=np.float32)
    if dtype == "bfloat16":
        q, k, v = _bf16_round(q), _bf16_round(k), _bf16_round(v)
    for b, n in enumerate(lens):
        k[b, :, n:] = 0.0
        v[b, :, n:] = 0.0
    h = hashlib.sha256()
    for a in (q, k, v):
        h.update(np.ascontiguousarray(a).tobytes())
    return dict(name=name, seed=seed, Hkv=hkv, G=g, lens=np.asarray(lens, np.int32), topk=topk, dtype=dtype,
                q=q, k=k, v=v, checksum=h.hexdigest(), local=local, sink=SINK if local is not None else 0)
