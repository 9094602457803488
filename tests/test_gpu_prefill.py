"""The causal prefill kernel over the paged cache against fp32 torch attention on the contiguous history.

Each case: sequences with some history already in their pages receive a chunk of new tokens
(ktk_append_tokens), then ktk_prefill_attention attends every new token to its own prefix.  Reference:
softmax(q K^T / sqrt(D)) V in fp32 with the causal mask over absolute positions -- what
flashinfer.single_prefill_with_kv_cache(causal=True) computes in LiteSys/litesys/attention/batch_cache.py:129-145.
"""
import math

import pytest
import torch

from helpers import paged_state, to_dev

pytestmark = pytest.mark.gpu


def _reference(q, k, v, G):
    """q [n_new, Hq, D], k/v [Hkv, total, D] fp32; new tokens are the last n_new positions."""
    n_new, Hq, D = q.shape
    total = k.shape[1]
    pos = torch.arange(total - n_new, total, device=q.device)
    mask = torch.arange(total, device=q.device)[None, :] <= pos[:, None]              # [n_new, total]
    kk = k.repeat_interleave(G, dim=0)                                                 # [Hq, total, D]
    vv = v.repeat_interleave(G, dim=0)
    logits = torch.einsum("nhd,htd->hnt", q, kk) / math.sqrt(D)
    logits = logits.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hnt,htd->nhd", torch.softmax(logits, dim=-1), vv)


@pytest.mark.parametrize("dtype,variant", [(torch.bfloat16, 0), (torch.bfloat16, 1), (torch.bfloat16, 2), (torch.bfloat16, 3),
                                           (torch.float32, 0)])
@pytest.mark.parametrize("G,Hkv,sink", [(4, 2, 0), (8, 1, 4), (2, 2, 4), (1, 3, 0)])
def test_prefill_matches_causal_attention(cuda_device, dtype, variant, G, Hkv, sink):
    from kinetics_b200 import ops
    # (history, new tokens): a fresh prompt, a chunk behind a long history, a chunk ending on a page edge, a
    # single new token, a prompt shorter than the sink, an empty chunk
    hist = [0, 300, 16 * 7 - 5 + sink, 77, 0, 40]
    new = [137, 61, 5, 1, 3, 0]
    B = len(hist)
    lens = [h + n for h, n in zip(hist, new)]
    g = torch.Generator().manual_seed(17 + G + sink)
    L = max(lens)
    k = torch.randn(B, Hkv, L, 128, generator=g).to(dtype).float()
    v = torch.randn(B, Hkv, L, 128, generator=g).to(dtype).float()
    # the pages hold only the history at first; the kernel under test's companion writes the chunk
    st = paged_state(k, v, lens, dtype, seed=3, sink=sink, fill=0.0)
    d = to_dev(st, cuda_device)
    status = ops.new_status(cuda_device)
    q_indptr = torch.tensor([sum(new[:i]) for i in range(B + 1)], dtype=torch.int32, device=cuda_device)
    total_new = sum(new)
    q = torch.randn(total_new, Hkv * G, 128, generator=g).to(dtype).to(cuda_device)
    view = ops.PageView(sink_tokens=sink, local_tokens=1) if sink else None
    # write the chunks again through the append kernel (the fixture already holds them: same bytes)
    k_new = torch.cat([k[b, :, hist[b]:lens[b]].transpose(0, 1) for b in range(B)]).to(dtype).to(cuda_device)
    v_new = torch.cat([v[b, :, hist[b]:lens[b]].transpose(0, 1) for b in range(B)]).to(dtype).to(cuda_device)
    before = d["kv_cache"].clone()
    ops.append_tokens(k_new.contiguous(), v_new.contiguous(), q_indptr, d["kv_cache"], None, d["kv_indices"],
                      d["kv_indptr"], d["kv_last_page_len"], status=status, view=view)
    assert torch.equal(before, d["kv_cache"])
    out = ops.prefill_attention(q, q_indptr, max(new), d["kv_cache"], d["kv_indices"], d["kv_indptr"],
                                d["kv_last_page_len"], variant=variant, status=status, view=view)
    ops.raise_on_status(status)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    for b in range(B):
        if new[b] == 0:
            continue
        lo, hi = int(q_indptr[b]), int(q_indptr[b + 1])
        ref = _reference(q[lo:hi].float(), k[b, :, :lens[b]].to(cuda_device), v[b, :, :lens[b]].to(cuda_device), G)
        torch.testing.assert_close(out[lo:hi].float(), ref, rtol=tol, atol=tol)


def test_prefill_long_prompt_many_sequences(cuda_device):
    # several 2000-token prompts in one launch, G = 4: tiles of 8 tokens, 126 pages for the last tile
    from kinetics_b200 import ops
    B, Hkv, G, n = 3, 2, 4, 2003
    g = torch.Generator().manual_seed(5)
    k = torch.randn(B, Hkv, n, 128, generator=g).to(torch.bfloat16).float()
    v = torch.randn(B, Hkv, n, 128, generator=g).to(torch.bfloat16).float()
    st = paged_state(k, v, [n] * B, torch.bfloat16, seed=4, fill=0.0)
    d = to_dev(st, cuda_device)
    q_indptr = torch.arange(B + 1, dtype=torch.int32, device=cuda_device) * n
    q = torch.randn(B * n, Hkv * G, 128, generator=g).to(torch.bfloat16).to(cuda_device)
    status = ops.new_status(cuda_device)
    out = ops.prefill_attention(q, q_indptr, n, d["kv_cache"], d["kv_indices"], d["kv_indptr"], d["kv_last_page_len"],
                                status=status)
    rows = ops.prefill_attention(q, q_indptr, n, d["kv_cache"], d["kv_indices"], d["kv_indptr"], d["kv_last_page_len"],
                                 variant=1, status=status)
    ops.raise_on_status(status)
    torch.testing.assert_close(out.float(), rows.float(), rtol=2e-2, atol=2e-2)
    ref = _reference(q[n:2 * n].float(), k[1].to(cuda_device), v[1].to(cuda_device), G)
    torch.testing.assert_close(out[n:2 * n].float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("variant", [0, 2])
@pytest.mark.parametrize("G,sink", [(4, 0), (2, 4), (8, 4)])
def test_prefill_on_block_and_tile_edges(cuda_device, variant, G, sink):
    """Histories and chunks that end exactly on the edges the kernels cut at: 16-token pages, the 64-key blocks
    and the 128 / G-token tiles of the tcgen05 kernel (and one token to either side of them)."""
    from kinetics_b200 import ops
    Hkv = 2
    tile = 128 // G
    hist = [0, 64 - sink, 64, 128 + sink, 63, 0, 16 * 9]
    new = [tile, tile, 2 * tile, tile + 1, 1, 64 + sink + 1, tile - 1]
    B = len(hist)
    lens = [h + n for h, n in zip(hist, new)]
    g = torch.Generator().manual_seed(40 + G + sink)
    L = max(lens)
    k = torch.randn(B, Hkv, L, 128, generator=g).to(torch.bfloat16).float()
    v = torch.randn(B, Hkv, L, 128, generator=g).to(torch.bfloat16).float()
    st = paged_state(k, v, lens, torch.bfloat16, seed=9, sink=sink)           # unused slots hold NaN
    d = to_dev(st, cuda_device)
    status = ops.new_status(cuda_device)
    q_indptr = torch.tensor([sum(new[:i]) for i in range(B + 1)], dtype=torch.int32, device=cuda_device)
    q = torch.randn(sum(new), Hkv * G, 128, generator=g).to(torch.bfloat16).to(cuda_device)
    view = ops.PageView(sink_tokens=sink, local_tokens=1) if sink else None
    out = ops.prefill_attention(q, q_indptr, max(new), d["kv_cache"], d["kv_indices"], d["kv_indptr"],
                                d["kv_last_page_len"], variant=variant, status=status, view=view)
    ops.raise_on_status(status)
    assert torch.isfinite(out.float()).all()
    for b in range(B):
        lo, hi = int(q_indptr[b]), int(q_indptr[b + 1])
        ref = _reference(q[lo:hi].float(), k[b, :, :lens[b]].to(cuda_device), v[b, :, :lens[b]].to(cuda_device), G)
        torch.testing.assert_close(out[lo:hi].float(), ref, rtol=2e-2, atol=2e-2)
