"""The function-level LiteSys chain (copy_to_cache -> qk -> attn_logits_processor -> softmax -> sv,
batch_cache.py:154-168) on the library's kernels, against the outputs the reference's own functions
produced for the golden cases (tests/golden/ls_*.npz) and against plain torch."""
import math

import numpy as np
import pytest
import torch

from helpers import LITESYS_CASES, LITESYS_TOKEN_CASES, load_golden, torch_dtype
from golden.cases import make_case

pytestmark = pytest.mark.gpu
SINK, BLOCK_SEQ = 4, 128


def _chain(cu, q, k_cache, v_cache, new_k, new_v, batch_idx, lengths_before, logits, sparse_kwargs, hq, hkv):
    """One decode step the way the reference's BatchKVManager.decode strings the functions together."""
    offset = lengths_before.clone()
    cu.copy_to_cache(k_cache, new_k, batch_idx, offset)
    cu.copy_to_cache(v_cache, new_v, batch_idx, offset)
    offset += 1
    cu.qk(query=q, key=k_cache, batch_idx=batch_idx, offset=offset, logits_buffer=logits, BLOCK_SEQ=BLOCK_SEQ)
    masked = cu.attn_logits_processor(logits, offset, hq, hkv, 1, **sparse_kwargs)
    kept_logits = masked.clone()
    cu.softmax(masked, batch_idx, offset)
    out = cu.sv(value=v_cache, batch_idx=batch_idx, offset=offset, logits_buffer=masked, output_buffer=None,
                BLOCK_SEQ=BLOCK_SEQ)
    return out, kept_logits


@pytest.mark.parametrize("name", sorted(LITESYS_CASES))
def test_function_chain_reproduces_the_reference_outputs(cuda_device, name):
    from kinetics_b200 import cache_utils as cu
    case, gold = make_case(name), load_golden(name)
    dt = torch_dtype(case["dtype"])
    lens = [int(n) for n in case["lens"]]
    B, hkv, g = len(lens), case["Hkv"], case["G"]
    hq, L = hkv * g, max(lens)
    max_len = (L + BLOCK_SEQ) // BLOCK_SEQ * BLOCK_SEQ
    k = torch.from_numpy(case["k"]).to(dt).to(cuda_device)            # [B, Hkv, L, D], the newest token included
    v = torch.from_numpy(case["v"]).to(dt).to(cuda_device)
    q = torch.from_numpy(case["q"]).to(dt).to(cuda_device).view(B, hq, 1, 128)
    k_cache = torch.zeros(B, hkv, max_len, 128, dtype=dt, device=cuda_device)
    v_cache = torch.zeros_like(k_cache)
    new_k = torch.empty(B, hkv, 1, 128, dtype=dt, device=cuda_device)
    new_v = torch.empty_like(new_k)
    for b, n in enumerate(lens):
        k_cache[b, :, :n - 1] = k[b, :, :n - 1]
        v_cache[b, :, :n - 1] = v[b, :, :n - 1]
        new_k[b, :, 0] = k[b, :, n - 1]
        new_v[b, :, 0] = v[b, :, n - 1]
    logits = torch.full((B, hq, max_len), float("-inf"), device=cuda_device)
    kwargs = cu.preprocess_sparse_args(attn_topk=None, attn_block_topk=case["topk"], attn_local=case["local"],
                                       attn_block_size=16)
    batch_idx = torch.arange(B, device=cuda_device)
    before = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=cuda_device)
    out, kept_logits = _chain(cu, q, k_cache, v_cache, new_k, new_v, batch_idx, before, logits, kwargs, hq, hkv)
    cu.check_status(cuda_device)
    # the appended token landed where the reference puts it
    for b, n in enumerate(lens):
        assert torch.equal(k_cache[b, :, n - 1], k[b, :, n - 1]) and torch.equal(v_cache[b, :, n - 1], v[b, :, n - 1])
    tol = 5e-5 if dt == torch.float32 else 2e-2
    np.testing.assert_allclose(out.float().cpu().numpy(), gold["out"], rtol=tol, atol=tol)
    # the blocks the mask kept are the ones the reference kept
    topk, local = case["topk"], case["local"]
    n_full = (SINK + local + topk * 16 + 15) // 16 * 16
    for b, n in enumerate(lens):
        if n <= n_full:
            continue
        nblk = (n - local - SINK) // 16
        region = kept_logits[b, :, SINK:SINK + nblk * 16].view(hkv, g, nblk, 16)
        alive = torch.isfinite(region).all(dim=3).all(dim=1)            # [Hkv, nblk]
        dead = torch.isinf(region).all(dim=3).all(dim=1)
        assert (alive | dead).all()
        for h in range(hkv):
            assert sorted(torch.nonzero(alive[h]).view(-1).tolist()) == sorted(int(x) for x in gold["kept"][b, h])
        # sink and tail untouched
        assert torch.isfinite(kept_logits[b, :, :SINK]).all() and torch.isfinite(kept_logits[b, :, SINK + nblk * 16:n]).all()


@pytest.mark.parametrize("name", sorted(LITESYS_TOKEN_CASES))
def test_function_chain_with_token_topk_reproduces_the_reference(cuda_device, name):
    # attn_topk: attn_logits_processor dispatches to topk_sparsity (sparsity_utils.py:6-21, :233-234)
    from kinetics_b200 import cache_utils as cu
    case, gold = make_case(name), load_golden(name)
    dt = torch_dtype(case["dtype"])
    lens = [int(n) for n in case["lens"]]
    B, hkv, g = len(lens), case["Hkv"], case["G"]
    hq, L = hkv * g, max(lens)
    max_len = (L + BLOCK_SEQ) // BLOCK_SEQ * BLOCK_SEQ
    k = torch.from_numpy(case["k"]).to(dt).to(cuda_device)
    v = torch.from_numpy(case["v"]).to(dt).to(cuda_device)
    q = torch.from_numpy(case["q"]).to(dt).to(cuda_device).view(B, hq, 1, 128)
    k_cache = torch.zeros(B, hkv, max_len, 128, dtype=dt, device=cuda_device)
    v_cache = torch.zeros_like(k_cache)
    new_k = torch.empty(B, hkv, 1, 128, dtype=dt, device=cuda_device)
    new_v = torch.empty_like(new_k)
    for b, n in enumerate(lens):
        k_cache[b, :, :n - 1] = k[b, :, :n - 1]
        v_cache[b, :, :n - 1] = v[b, :, :n - 1]
        new_k[b, :, 0] = k[b, :, n - 1]
        new_v[b, :, 0] = v[b, :, n - 1]
    logits = torch.full((B, hq, max_len), float("-inf"), device=cuda_device)
    topk, local = case["topk"], case["local"]
    kwargs = cu.preprocess_sparse_args(attn_topk=topk, attn_local=local)
    batch_idx = torch.arange(B, device=cuda_device)
    before = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=cuda_device)
    out, kept_logits = _chain(cu, q, k_cache, v_cache, new_k, new_v, batch_idx, before, logits, kwargs, hq, hkv)
    cu.check_status(cuda_device)
    tol = 5e-5 if dt == torch.float32 else 2e-2
    np.testing.assert_allclose(out.float().cpu().numpy(), gold["out"], rtol=tol, atol=tol)
    # the positions the mask kept are the reference's, for every head of a group alike
    for b, n in enumerate(lens):
        fin = torch.isfinite(kept_logits[b, :, :n]).view(hkv, g, n)
        assert (fin == fin[:, :1]).all()
        if n <= SINK + topk + local:
            assert fin.all()
            continue
        assert fin[:, :, :SINK].all() and fin[:, :, n - local:].all()
        for h in range(hkv):
            pos = (torch.nonzero(fin[h, 0, SINK:n - local]).view(-1) + SINK).tolist()
            assert pos == [int(x) for x in gold["kept"][b, h]], (name, b, h)


def test_token_topk_mask_ties_go_to_the_lower_position(cuda_device):
    from kinetics_b200 import cache_utils as cu
    hq, hkv, n, topk, local = 4, 2, 200, 5, 3
    logits = torch.zeros(1, hq, 256, device=cuda_device)              # every dynamic token ties
    logits[0, :, 50] = 1.0                                            # one clear winner
    off = torch.tensor([n], dtype=torch.int32, device=cuda_device)
    cu.topk_sparsity(logits, off, hq, hkv, topk, local, sink=SINK)
    cu.check_status(cuda_device)
    kept = torch.nonzero(torch.isfinite(logits[0, 0, SINK:n - local])).view(-1).tolist()
    assert kept == [0, 1, 2, 3, 46]                                   # positions 4..7 and 50
    assert torch.isfinite(logits[0, :, :SINK]).all() and torch.isfinite(logits[0, :, n - local:n]).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dense_chain_with_scattered_slots(cuda_device, dtype):
    # no sparsity; rows of the active batch live in arbitrary cache slots
    from kinetics_b200 import cache_utils as cu
    g = torch.Generator().manual_seed(3)
    B, hkv, grp, max_batch, max_len = 4, 2, 4, 7, 640
    hq = hkv * grp
    lens = [1, 130, 600, 17]
    slots = [5, 0, 6, 2]
    k_cache = torch.randn(max_batch, hkv, max_len, 128, generator=g).to(dtype).to(cuda_device)
    v_cache = torch.randn(max_batch, hkv, max_len, 128, generator=g).to(dtype).to(cuda_device)
    q = torch.randn(B, hq, 1, 128, generator=g).to(dtype).to(cuda_device)
    new_k = torch.randn(B, hkv, 1, 128, generator=g).to(dtype).to(cuda_device)
    new_v = torch.randn(B, hkv, 1, 128, generator=g).to(dtype).to(cuda_device)
    logits = torch.full((max_batch, hq, max_len), float("-inf"), device=cuda_device)
    batch_idx = torch.tensor(slots, device=cuda_device)
    before = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=cuda_device)
    kwargs = cu.preprocess_sparse_args()
    out, _ = _chain(cu, q, k_cache, v_cache, new_k, new_v, batch_idx, before, logits, kwargs, hq, hkv)
    cu.check_status(cuda_device)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for b, (n, s) in enumerate(zip(lens, slots)):
        kk = k_cache[s, :, :n].float().repeat_interleave(grp, 0)        # [Hq, n, D], the new token included
        vv = v_cache[s, :, :n].float().repeat_interleave(grp, 0)
        assert torch.equal(k_cache[s, :, n - 1], new_k[b, :, 0])
        p = torch.softmax(torch.einsum("hd,hnd->hn", q[b, :, 0].float(), kk) / math.sqrt(128), -1)
        ref = torch.einsum("hn,hnd->hd", p, vv)
        torch.testing.assert_close(out[b].float(), ref, rtol=tol, atol=tol)
        # qk wrote -inf behind the sequence up to the end of its last 128-block and nothing beyond
        end = (n + BLOCK_SEQ - 1) // BLOCK_SEQ * BLOCK_SEQ
        assert torch.isinf(logits[b, :, n:end]).all()


def test_other_masks_are_refused(cuda_device):
    from kinetics_b200 import cache_utils as cu
    logits = torch.zeros(1, 4, 128, device=cuda_device)
    off = torch.tensor([100], dtype=torch.int32, device=cuda_device)
    with pytest.raises(NotImplementedError):
        cu.attn_logits_processor(logits, off, 4, 1, 1, **cu.preprocess_sparse_args(attn_random_select=8, attn_local=4,
                                                                                   attn_topk=None))
    # layer 0 is skipped by default, whatever the mask
    assert cu.attn_logits_processor(logits, off, 4, 1, 0, **cu.preprocess_sparse_args(attn_topk=8, attn_local=4)) is logits
