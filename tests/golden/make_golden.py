"""Generate tests/golden/*.npz by running the REFERENCE's own Python on CPU.

Run once in a container that has the reference checkout (it is not needed afterwards):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py <path to the Kinetics checkout>

What runs is the reference's LiteSys decode chain, unmodified, imported from its checkout:
``qk`` -> ``blockwise_topk_sparsity`` -> ``softmax`` -> ``sv``
(LiteSys/litesys/attention/cache_utils.py, sparsity_utils.py), the Triton kernels under the
Triton interpreter.  ``blockwise_topk_sparsity`` is called with ``sink=0, local=1,
block_size=16``: the dynamic region is then every full 16-token block in front of the block
holding the newest token, and that last block is always kept -- exactly the paged block
top-k of benchmark/blocktopk_decoder.py:216-221 (n scored pages + the page being filled).

Stored per case: the attention output, the set of kept blocks per (sequence, kv head), and
the margin between the k-th and (k+1)-th block score (cases with a near tie are rejected, so
that the stored set does not depend on summation order).
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from cases import CASES, LITESYS_CASES, LITESYS_TOKEN_CASES, SINK, D, P, make_case  # noqa: E402


def run_reference(ref_root: str, case: dict) -> dict:
    sys.path.insert(0, os.path.join(ref_root, "LiteSys"))
    from litesys.attention.cache_utils import qk, softmax, sv
    from litesys.attention.sparsity_utils import blockwise_topk_sparsity

    hkv, g, topk = case["Hkv"], case["G"], case["topk"]
    hq = hkv * g
    lens = torch.from_numpy(case["lens"])
    B, L = len(lens), int(lens.max())
    max_len = (L + 127) // 128 * 128
    # The Triton interpreter has no bf16 constants, so the reference kernels always run on fp32
    # tensors; a "bfloat16" case holds bf16-representable values, which fp32 carries exactly.
    tdt = torch.float32
    k_cache = torch.zeros(B, hkv, max_len, D, dtype=tdt)
    v_cache = torch.zeros(B, hkv, max_len, D, dtype=tdt)
    k_cache[:, :, :L] = torch.from_numpy(case["k"]).to(tdt)
    v_cache[:, :, :L] = torch.from_numpy(case["v"]).to(tdt)
    query = torch.from_numpy(case["q"]).to(tdt).view(B, hq, 1, D)
    batch_idx = torch.arange(B, dtype=torch.long)
    offset = lens.to(torch.int32)
    logits = torch.full((B, hq, max_len), float("-inf"), dtype=torch.float32)
    nblk = (max_len + 127) // 128
    out_buf = torch.zeros(B, hq, nblk, D, dtype=torch.float32)

    qk(query=query, key=k_cache, batch_idx=batch_idx, offset=offset, logits_buffer=logits, BLOCK_SEQ=128)
    dense_logits = logits.clone()
    logits = blockwise_topk_sparsity(logits, offset, hq, hkv, topk, 1, sink=0, block_size=P)
    masked = logits.clone()
    softmax(logits, batch_idx, offset)
    out = sv(value=v_cache, batch_idx=batch_idx, offset=offset, logits_buffer=logits, output_buffer=out_buf,
             BLOCK_SEQ=128)

    kept = np.full((B, hkv, topk), -1, np.int32)
    margin = np.full((B, hkv), np.inf, np.float64)
    for b in range(B):
        n = int(lens[b])
        n_scored = (n - 1) // P
        for h in range(hkv):
            fin = torch.isfinite(masked[b, h * g, : n_scored * P]).view(n_scored, P)
            assert bool((fin.all(1) | (~fin).all(1)).all()), "a block is partly masked"
            blocks = torch.nonzero(fin[:, 0]).flatten().numpy() if n_scored else np.zeros(0, np.int64)
            if n_scored > topk:
                assert len(blocks) == topk, (b, h, len(blocks))
                kept[b, h] = np.sort(blocks)
                # margin of the decision, in float64, relative to the score spread
                sc = dense_logits[b, h * g:(h + 1) * g, : n_scored * P].double().mean(0).view(n_scored, P).mean(1)
                srt = torch.sort(sc, descending=True).values
                margin[b, h] = float((srt[topk - 1] - srt[topk]) / (srt[0] - srt[-1]))
            else:
                assert len(blocks) == n_scored
                kept[b, h, :n_scored] = blocks
    need = 2e-2 if case["dtype"] == "bfloat16" else 1e-5
    assert margin.min() > need, f"near tie in case {case['name']}: margin {margin.min():.3g}; change the seed"
    return dict(out=out.float().numpy().reshape(B, hq, D), kept=kept, margin=margin)


def run_reference_litesys(ref_root: str, case: dict) -> dict:
    """The LiteSys decode chain exactly as BatchKVManager.decode runs it (batch_cache.py:154-168):
    qk -> attn_logits_processor(**preprocess_sparse_args(attn_block_topk, attn_local, attn_block_size))
    -> softmax -> sv, for a layer that is not in attn_layer_skip.  Defaults of the reference: sink = 4."""
    sys.path.insert(0, os.path.join(ref_root, "LiteSys"))
    from litesys.attention.cache_utils import qk, softmax, sv
    from litesys.attention.sparsity_utils import attn_logits_processor, preprocess_sparse_args

    hkv, g, topk, local = case["Hkv"], case["G"], case["topk"], case["local"]
    hq = hkv * g
    lens = torch.from_numpy(case["lens"])
    B, L = len(lens), int(lens.max())
    max_len = (L + 127) // 128 * 128
    k_cache = torch.zeros(B, hkv, max_len, D)
    v_cache = torch.zeros(B, hkv, max_len, D)
    k_cache[:, :, :L] = torch.from_numpy(case["k"])
    v_cache[:, :, :L] = torch.from_numpy(case["v"])
    query = torch.from_numpy(case["q"]).view(B, hq, 1, D)
    batch_idx = torch.arange(B, dtype=torch.long)
    offset = lens.to(torch.int32)
    logits = torch.full((B, hq, max_len), float("-inf"), dtype=torch.float32)
    out_buf = torch.zeros(B, hq, (max_len + 127) // 128, D, dtype=torch.float32)
    kwargs = preprocess_sparse_args(attn_topk=None, attn_block_topk=topk, attn_local=local, attn_block_size=P)

    qk(query=query, key=k_cache, batch_idx=batch_idx, offset=offset, logits_buffer=logits, BLOCK_SEQ=128)
    dense_logits = logits.clone()
    logits = attn_logits_processor(logits, offset, hq, hkv, 1, **kwargs)
    masked = logits.clone()
    softmax(logits, batch_idx, offset)
    out = sv(value=v_cache, batch_idx=batch_idx, offset=offset, logits_buffer=logits, output_buffer=out_buf,
             BLOCK_SEQ=128)

    kept = np.full((B, hkv, topk), -1, np.int32)
    margin = np.full((B, hkv), np.inf, np.float64)
    n_full = (SINK + local + topk * P + P - 1) // P * P          # sparsity_utils.py:27-28
    for b in range(B):
        n = int(lens[b])
        n_dyn = max(0, n - local - SINK) // P
        for h in range(hkv):
            fin = torch.isfinite(masked[b, h * g, SINK: SINK + n_dyn * P]).view(n_dyn, P)
            assert bool((fin.all(1) | (~fin).all(1)).all()), "a block is partly masked"
            blocks = torch.nonzero(fin[:, 0]).flatten().numpy() if n_dyn else np.zeros(0, np.int64)
            assert bool(torch.isfinite(masked[b, h * g, :min(SINK, n)]).all())           # the sink is kept
            assert bool(torch.isfinite(masked[b, h * g, SINK + n_dyn * P: n]).all())     # so is the tail
            if n > n_full:
                assert len(blocks) == topk, (b, h, len(blocks))
                kept[b, h] = np.sort(blocks)
                sc = dense_logits[b, h * g:(h + 1) * g, SINK: SINK + n_dyn * P].double().mean(0).view(n_dyn, P).mean(1)
                srt = torch.sort(sc, descending=True).values
                if n_dyn > topk:
                    margin[b, h] = float((srt[topk - 1] - srt[topk]) / (srt[0] - srt[-1]))
            else:
                assert len(blocks) == n_dyn
                kept[b, h, :min(n_dyn, topk)] = blocks[:topk]
                assert n_dyn <= topk
    need = 2e-2 if case["dtype"] == "bfloat16" else 1e-4
    assert margin.min() > need, f"near tie in case {case['name']}: margin {margin.min():.3g}; change the seed"
    return dict(out=out.float().numpy().reshape(B, hq, D), kept=kept, margin=margin)


def run_reference_litesys_token(ref_root: str, case: dict) -> dict:
    """The same chain with the token-level mask: attn_logits_processor(**preprocess_sparse_args(attn_topk,
    attn_local)) dispatches to topk_sparsity (sparsity_utils.py:6-21, :233-234)."""
    sys.path.insert(0, os.path.join(ref_root, "LiteSys"))
    from litesys.attention.cache_utils import qk, softmax, sv
    from litesys.attention.sparsity_utils import attn_logits_processor, preprocess_sparse_args

    hkv, g, topk, local = case["Hkv"], case["G"], case["topk"], case["local"]
    hq = hkv * g
    lens = torch.from_numpy(case["lens"])
    B, L = len(lens), int(lens.max())
    max_len = (L + 127) // 128 * 128
    k_cache = torch.zeros(B, hkv, max_len, D)
    v_cache = torch.zeros(B, hkv, max_len, D)
    k_cache[:, :, :L] = torch.from_numpy(case["k"])
    v_cache[:, :, :L] = torch.from_numpy(case["v"])
    query = torch.from_numpy(case["q"]).view(B, hq, 1, D)
    batch_idx = torch.arange(B, dtype=torch.long)
    offset = lens.to(torch.int32)
    logits = torch.full((B, hq, max_len), float("-inf"), dtype=torch.float32)
    out_buf = torch.zeros(B, hq, (max_len + 127) // 128, D, dtype=torch.float32)
    kwargs = preprocess_sparse_args(attn_topk=topk, attn_local=local)

    qk(query=query, key=k_cache, batch_idx=batch_idx, offset=offset, logits_buffer=logits, BLOCK_SEQ=128)
    dense_logits = logits.clone()
    logits = attn_logits_processor(logits, offset, hq, hkv, 1, **kwargs)
    masked = logits.clone()
    softmax(logits, batch_idx, offset)
    out = sv(value=v_cache, batch_idx=batch_idx, offset=offset, logits_buffer=logits, output_buffer=out_buf,
             BLOCK_SEQ=128)

    kept = np.full((B, hkv, topk), -1, np.int32)           # kept positions of the dynamic region, ascending
    margin = np.full((B, hkv), np.inf, np.float64)
    for b in range(B):
        n = int(lens[b])
        for h in range(hkv):
            fin = torch.isfinite(masked[b, h * g, :n])
            for gg in range(1, g):
                assert torch.equal(fin, torch.isfinite(masked[b, h * g + gg, :n])), "heads of a group differ"
            if n > SINK + topk + local:                     # sparsity_utils.py:9,12
                assert bool(fin[:SINK].all()) and bool(fin[n - local:].all())
                pos = torch.nonzero(fin[SINK:n - local]).flatten().numpy() + SINK
                assert len(pos) == topk, (b, h, len(pos))
                kept[b, h] = pos
                sc = dense_logits[b, h * g:(h + 1) * g, SINK:n - local].double().mean(0)
                srt = torch.sort(sc, descending=True).values
                margin[b, h] = float((srt[topk - 1] - srt[topk]) / (srt[0] - srt[-1]))
            else:
                assert bool(fin.all())
    assert margin.min() > 1e-6, f"near tie in case {case['name']}: margin {margin.min():.3g}; change the seed"
    return dict(out=out.float().numpy().reshape(B, hq, D), kept=kept, margin=margin)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to the Kinetics checkout>")
    ref_root = sys.argv[1]
    for name in CASES:
        case = make_case(name)
        res = run_reference(ref_root, case)
        np.savez_compressed(HERE / f"{name}.npz", out=res["out"], kept=res["kept"], margin=res["margin"],
                            lens=case["lens"], topk=case["topk"], Hkv=case["Hkv"], G=case["G"],
                            checksum=case["checksum"], dtype=case["dtype"])
        print(f"{name}: out {res['out'].shape} min margin {res['margin'].min():.3g}")
    for name in LITESYS_CASES:
        case = make_case(name)
        res = run_reference_litesys(ref_root, case)
        np.savez_compressed(HERE / f"{name}.npz", out=res["out"], kept=res["kept"], margin=res["margin"],
                            lens=case["lens"], topk=case["topk"], Hkv=case["Hkv"], G=case["G"], local=case["local"],
                            sink=SINK, checksum=case["checksum"], dtype=case["dtype"])
        print(f"{name}: out {res['out'].shape} min margin {res['margin'].min():.3g}")
    for name in LITESYS_TOKEN_CASES:
        case = make_case(name)
        res = run_reference_litesys_token(ref_root, case)
        np.savez_compressed(HERE / f"{name}.npz", out=res["out"], kept=res["kept"], margin=res["margin"],
                            lens=case["lens"], topk=case["topk"], Hkv=case["Hkv"], G=case["G"], local=case["local"],
                            sink=SINK, checksum=case["checksum"], dtype=case["dtype"])
        print(f"{name}: out {res['out'].shape} min margin {res['margin'].min():.3g}")


if __name__ == "__main__":
    main()
