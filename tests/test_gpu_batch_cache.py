"""BatchKVManager (LiteSys interface) on the GPU against the oracle under the LiteSys page view."""
import math

import numpy as np
import pytest
import torch

from helpers import paged_state
from oracle import oracle

pytestmark = pytest.mark.gpu
SINK = 4


class Cfg:
    hidden_size = 1024
    num_attention_heads = 8
    num_key_value_heads = 2
    head_dim = 128
    num_hidden_layers = 2


def _oracle_step(hist_k, hist_v, q, lens, dtype, topk, local, dense):
    """hist_k/v [B, Hkv, L, D] fp32 histories (already holding the newest token); q [B, Hq, D]."""
    st = paged_state(hist_k, hist_v, lens, dtype, seed=1, sink=SINK)
    if dense:
        return oracle.decode_v(q, st["kv_cache"], st["kv_indices"], -1, st["kv_indptr"], st["kv_last_page_len"],
                               1 / math.sqrt(128), SINK, local)
    summ = oracle.summaries_v(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"],
                              st["summary_stride"], SINK)
    phys, _, _ = oracle.select_v(q, summ, st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"], topk, SINK, local)
    return oracle.decode_v(q, st["kv_cache"], phys, topk, st["kv_indptr"], st["kv_last_page_len"],
                           1 / math.sqrt(128), SINK, local)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_prefill_then_decode_matches_the_litesys_semantics(cuda_device, dtype):
    from kinetics_b200 import BatchKVManager
    topk, local = 3, 7
    mgr = BatchKVManager(Cfg, max_batch_size=6, max_seq_len=512, device=cuda_device, dtype=dtype,
                         attn_block_topk=topk, attn_local=local, attn_block_size=16)
    g = torch.Generator().manual_seed(0)
    slots, plens = [2, 0, 5], [150, 37, 3]
    L = 512
    hist_k = torch.zeros(2, 6, 2, L, 128)           # [layer, slot, Hkv, L, D]
    hist_v = torch.zeros(2, 6, 2, L, 128)
    lens = {s: 0 for s in range(6)}
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4

    def rnd(*shape):
        return torch.randn(*shape, generator=g).to(dtype).float()

    # ---- prefill, one sequence at a time, in two chunks for the first one (append behind a prefix)
    for slot, n in zip(slots, plens):
        chunks = [n] if slot != 2 else [100, 50]
        for c in chunks:
            for layer in range(2):
                q, k, v = rnd(1, 8, c, 128), rnd(1, 2, c, 128), rnd(1, 2, c, 128)
                off = lens[slot]
                hist_k[layer, slot, :, off:off + c] = k[0]
                hist_v[layer, slot, :, off:off + c] = v[0]
                out = mgr.compute_attention(q.to(dtype).to(cuda_device), k.to(dtype).to(cuda_device),
                                            v.to(dtype).to(cuda_device), layer, torch.tensor([slot], device=cuda_device))
                tot = off + c
                kk = hist_k[layer, slot, :, :tot].repeat_interleave(4, 0)
                vv = hist_v[layer, slot, :, :tot].repeat_interleave(4, 0)
                logits = torch.einsum("hsd,htd->hst", q[0], kk) / math.sqrt(128)
                mask = torch.arange(tot)[None, :] <= (off + torch.arange(c))[:, None]
                ref = torch.softmax(logits.masked_fill(~mask, float("-inf")), -1) @ vv
                np.testing.assert_allclose(out.float().cpu().numpy().reshape(c, 8, 128),
                                           ref.transpose(0, 1).numpy(), rtol=tol, atol=tol)
            lens[slot] += c
    mgr.check_status()

    # ---- decode steps over non-contiguous active slots; layer 0 stays dense (attn_layer_skip default)
    batch_idx = torch.tensor(slots, device=cuda_device)
    for step in range(20):
        for layer in range(2):
            q, k, v = rnd(3, 8, 1, 128), rnd(3, 2, 1, 128), rnd(3, 2, 1, 128)
            for i, s in enumerate(slots):
                hist_k[layer, s, :, lens[s]] = k[i, :, 0]
                hist_v[layer, s, :, lens[s]] = v[i, :, 0]
            out = mgr.compute_attention(q.to(dtype).to(cuda_device), k.to(dtype).to(cuda_device),
                                        v.to(dtype).to(cuda_device), layer, batch_idx)
            now = [lens[s] + 1 for s in slots]
            ref = _oracle_step(hist_k[layer, slots], hist_v[layer, slots], q[:, :, 0].to(dtype), now, dtype, topk,
                               local, dense=(layer == 0))
            assert out.shape == (3, 1, 8 * 128)
            np.testing.assert_allclose(out.float().cpu().numpy().reshape(3, 8, 128), ref.numpy(), rtol=tol, atol=tol)
        for s in slots:
            lens[s] += 1
    mgr.check_status()
    assert mgr.kv_offset[1][torch.tensor(slots, device=cuda_device)].tolist() == [lens[s] for s in slots]

    # ---- a cleared slot starts again from nothing
    mgr.clear_cache(0)
    assert int(mgr.kv_offset[0][0]) == 0 and int(mgr.kv_offset[1][0]) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_token_topk_decode_matches_the_reference_chain(cuda_device, dtype):
    # attn_topk (sparsity_utils.py:6-21) on the paged manager: prefill, then decode steps over scattered slots,
    # against the oracle's restatement of qk -> topk_sparsity -> softmax -> sv (pinned by tests/golden/ls_tok_*)
    from kinetics_b200 import BatchKVManager
    topk, local = 24, 5
    mgr = BatchKVManager(Cfg, max_batch_size=5, max_seq_len=384, device=cuda_device, dtype=dtype,
                         attn_topk=topk, attn_local=local)
    g = torch.Generator().manual_seed(4)
    slots, plens = [3, 0, 4], [200, SINK + topk + local - 2, 2]       # the second crosses the threshold while decoding
    L = 384
    hist_k = torch.zeros(2, 5, 2, L, 128)
    hist_v = torch.zeros(2, 5, 2, L, 128)
    lens = {s: 0 for s in range(5)}
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4

    def rnd(*shape):
        return torch.randn(*shape, generator=g).to(dtype).float()

    for slot, n in zip(slots, plens):
        for layer in range(2):
            q, k, v = rnd(1, 8, n, 128), rnd(1, 2, n, 128), rnd(1, 2, n, 128)
            hist_k[layer, slot, :, :n] = k[0]
            hist_v[layer, slot, :, :n] = v[0]
            mgr.compute_attention(q.to(dtype).to(cuda_device), k.to(dtype).to(cuda_device),
                                  v.to(dtype).to(cuda_device), layer, torch.tensor([slot], device=cuda_device))
        lens[slot] = n
    batch_idx = torch.tensor(slots, device=cuda_device)
    for step in range(6):
        for layer in range(2):
            q, k, v = rnd(3, 8, 1, 128), rnd(3, 2, 1, 128), rnd(3, 2, 1, 128)
            for i, s in enumerate(slots):
                hist_k[layer, s, :, lens[s]] = k[i, :, 0]
                hist_v[layer, s, :, lens[s]] = v[i, :, 0]
            out = mgr.compute_attention(q.to(dtype).to(cuda_device), k.to(dtype).to(cuda_device),
                                        v.to(dtype).to(cuda_device), layer, batch_idx)
            now = [lens[s] + 1 for s in slots]
            # layer 0 is in attn_layer_skip by default (dense): a budget that covers everything
            ref, kept = oracle.token_topk_decode(q[:, :, 0], hist_k[layer, slots], hist_v[layer, slots], now,
                                                 topk if layer else 10 ** 6, local, SINK, 1 / math.sqrt(128))
            torch.testing.assert_close(out.float().cpu().view(3, 8, 128), ref, rtol=tol, atol=tol)
            if layer == 1 and step == 5:
                assert (kept[0] >= 0).all() and (kept[1] >= 0).all() and (kept[2] < 0).all()
        for s in slots:
            lens[s] += 1
    mgr.check_status()


def test_unbuilt_masks_are_refused():
    from kinetics_b200 import BatchKVManager
    with pytest.raises(NotImplementedError):
        BatchKVManager(Cfg, 2, 128, "cuda", torch.bfloat16, attn_random_select=64, attn_local=16)
    with pytest.raises(NotImplementedError):
        BatchKVManager(Cfg, 2, 128, "cuda", torch.bfloat16, attn_local=16)
