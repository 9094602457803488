"""The CPU oracle against the vectors the reference's own Python produced (tests/golden)."""
import numpy as np
import pytest
import torch

from helpers import CASES, LITESYS_CASES, LITESYS_TOKEN_CASES, P, SINK, case_state, load_golden, make_case
from oracle import oracle


@pytest.mark.parametrize("name", sorted(CASES))
def test_inputs_match_fixture(name):
    case, _, _ = case_state(name)
    gold = load_golden(name)
    assert str(gold["checksum"]) == case["checksum"], "input generator drifted: regenerate the goldens"


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_reference(name):
    case, st, q = case_state(name, seed=11)
    gold = load_golden(name)
    topk = int(gold["topk"])
    summ = oracle.summaries(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"],
                            st["summary_stride"])
    phys, logical = oracle.select(q, summ, st["kv_indices"], st["kv_indptr"], topk)
    B, Hkv = logical.shape[:2]
    for b in range(B):
        n_scored = st["npages"][b] - 1
        cnt = min(topk, n_scored)
        for h in range(Hkv):
            mine = logical[b, h, :cnt].numpy()
            ref = gold["kept"][b, h][gold["kept"][b, h] >= 0]
            assert np.array_equal(np.sort(mine), ref), (name, b, h)
            assert logical[b, h, cnt] == st["npages"][b] - 1          # the page being filled
            assert (logical[b, h, cnt + 1:] == -1).all()
            table = st["kv_indices"][st["kv_indptr"][b]:st["kv_indptr"][b + 1]]
            assert torch.equal(phys[b, h, :cnt + 1], table[logical[b, h, :cnt + 1].long()])
    out = oracle.decode(q, st["kv_cache"], phys, topk, st["kv_indptr"], st["kv_last_page_len"],
                        oracle.default_scale())
    tol = 1e-4 if case["dtype"] == "float32" else 2e-2
    np.testing.assert_allclose(out.numpy(), gold["out"], rtol=tol, atol=tol)
    # the reference computed in fp32 on the same values: agreement is in fact far tighter
    assert np.abs(out.numpy() - gold["out"]).max() < 5e-5


def test_descending_order_and_tie_break():
    # equal summaries -> equal scores -> the lowest pages win, in ascending page order
    B, Hkv, G, n, topk = 1, 1, 4, 40, 5
    q = torch.randn(B, Hkv * G, 128)
    summ = torch.ones(B, Hkv, n + 1, 128)
    indptr = torch.tensor([0, n + 1], dtype=torch.int32)
    indices = torch.arange(100, 100 + n + 1, dtype=torch.int32)
    phys, logical = oracle.select(q, summ, indices, indptr, topk)
    assert logical[0, 0].tolist() == [0, 1, 2, 3, 4, n]
    assert phys[0, 0].tolist() == [100, 101, 102, 103, 104, 100 + n]
    # distinct scores come back largest first
    summ = torch.randn(B, Hkv, n + 1, 128)
    sc = oracle.scores(q, summ, indptr)
    _, logical = oracle.select_from_scores(sc, indices, indptr, topk)
    picked = sc[0, 0, logical[0, 0, :topk].long()]
    assert (picked[:-1] >= picked[1:]).all()
    rest = torch.ones(n, dtype=torch.bool)
    rest[logical[0, 0, :topk].long()] = False
    assert picked[-1] >= sc[0, 0, :n][rest].max()


def test_negative_zero_ties_with_zero():
    sc = torch.tensor([[[0.0, -0.0, -0.0, 0.0, -1.0, 0.0]]])
    indptr = torch.tensor([0, 6], dtype=torch.int32)   # 5 scored pages + the last one
    indices = torch.arange(6, dtype=torch.int32)
    _, logical = oracle.select_from_scores(sc, indices, indptr, 3)
    assert logical[0, 0].tolist() == [0, 1, 2, 5]


def test_scores_match_float64_closely():
    torch.manual_seed(3)
    B, Hkv, G, n = 2, 2, 4, 33
    q = torch.randn(B, Hkv * G, 128)
    summ = torch.randn(B, Hkv, n, 128)
    indptr = torch.tensor([0, n + 1, 2 * n + 2], dtype=torch.int32)
    sc = oracle.scores(q, summ, indptr)
    ref = torch.einsum("bhgd,bhnd->bhn", q.view(B, Hkv, G, 128).double(), summ.double()) / G
    assert torch.allclose(sc.double(), ref, atol=2e-5, rtol=1e-5)


def test_incremental_append_equals_bulk_summaries():
    torch.manual_seed(5)
    B, Hkv, steps = 3, 2, 37
    for dt in (torch.float32, torch.bfloat16):
        total = B * 4
        cache = torch.zeros(total, 2, P, Hkv, 128, dtype=dt)
        summ = torch.zeros(B, Hkv, 4, 128, dtype=dt)
        table = torch.randperm(total).view(B, 4).to(torch.int32)
        for s in range(steps):
            npg = s // P + 1
            indices = table[:, :npg].contiguous().view(-1)
            indptr = (torch.arange(B + 1) * npg).to(torch.int32)
            last = torch.full((B,), s % P + 1, dtype=torch.int32)
            k = torch.randn(B, Hkv, 128).to(dt)
            v = torch.randn(B, Hkv, 128).to(dt)
            oracle.append(k, v, cache, summ, indices, indptr, last)
        bulk = oracle.summaries(cache, indices, indptr, last, 4)
        assert torch.equal(bulk.view(torch.int16 if dt == torch.bfloat16 else torch.int32),
                           summ.view(torch.int16 if dt == torch.bfloat16 else torch.int32))


def test_reference_torch_lines_agree_with_oracle_selection():
    # benchmark/blocktopk_decoder.py:216-217 in fp32 picks the same page SET (no near ties here)
    case, st, q = case_state("cfg1_fp32", seed=2)
    topk = case["topk"]
    summ = oracle.summaries(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"],
                            st["summary_stride"])
    phys, _ = oracle.select(q, summ, st["kv_indices"], st["kv_indptr"], topk)
    B = q.shape[0]
    n = st["npages"][0] - 1
    table = st["kv_indices"].view(B, n + 1)
    ref = oracle.reference_torch_select(q.view(B, 4, 128), summ[:, 0, :n], table, topk)
    assert torch.equal(torch.sort(ref[:, :topk].long(), 1).values, torch.sort(phys[:, 0, :topk].long(), 1).values)
    assert torch.equal(ref[:, topk], phys[:, 0, topk])
    out_ref = oracle.reference_torch_decode(q.view(B, 4, 128), st["kv_cache"], ref, 1, oracle.default_scale())
    out = oracle.decode(q, st["kv_cache"], phys, topk, st["kv_indptr"], st["kv_last_page_len"],
                        oracle.default_scale())
    assert torch.allclose(out_ref, out, atol=1e-5, rtol=1e-5)


# ---------------------------------------------------------------- LiteSys semantics (sink 4, local window)

@pytest.mark.parametrize("name", sorted(LITESYS_CASES))
def test_oracle_view_reproduces_litesys_chain(name):
    """qk -> attn_logits_processor(blockwise top-k) -> softmax -> sv of the reference, run on CPU when the
    fixtures were made, against the oracle under the view (sink_tokens=4, local_tokens=attn_local)."""
    case, st, q = case_state(name, seed=13)
    gold = load_golden(name)
    assert str(gold["checksum"]) == case["checksum"]
    topk, local = int(gold["topk"]), int(gold["local"])
    summ = oracle.summaries_v(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"],
                              st["summary_stride"], SINK)
    phys, logical, _ = oracle.select_v(q, summ, st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"], topk,
                                       SINK, local)
    B, Hkv = logical.shape[:2]
    for b in range(B):
        n = int(case["lens"][b])
        n_dyn = max(0, n - local - SINK) // P
        for h in range(Hkv):
            row = logical[b, h][logical[b, h] >= 0].numpy()
            assert row[0] == 0                                   # the sink page
            picks = row[(row >= 1) & (row < 1 + n_dyn)] - 1      # scored pages <-> reference blocks
            ref = gold["kept"][b, h][gold["kept"][b, h] >= 0]
            assert np.array_equal(np.sort(picks), ref), (name, b, h)
            tail = row[row >= 1 + n_dyn]
            assert np.array_equal(tail, np.arange(1 + n_dyn, st["npages"][b]))   # everything after them
    out = oracle.decode_v(q, st["kv_cache"], phys, topk, st["kv_indptr"], st["kv_last_page_len"],
                          oracle.default_scale(), SINK, local)
    assert np.abs(out.numpy() - gold["out"]).max() < 5e-5
    dense = oracle.decode_v(q, st["kv_cache"], st["kv_indices"], -1, st["kv_indptr"], st["kv_last_page_len"],
                            oracle.default_scale(), SINK, local)
    assert torch.isfinite(dense).all()


@pytest.mark.parametrize("name", sorted(LITESYS_TOKEN_CASES))
def test_oracle_token_topk_reproduces_litesys_chain(name):
    """qk -> attn_logits_processor(attn_topk) -> softmax -> sv of the reference (topk_sparsity,
    sparsity_utils.py:6-21), run on CPU when the fixtures were made, against the oracle's token-level restatement."""
    case = make_case(name)
    gold = load_golden(name)
    assert str(gold["checksum"]) == case["checksum"]
    topk, local = int(gold["topk"]), int(gold["local"])
    q, k, v = (torch.from_numpy(case[x]) for x in ("q", "k", "v"))
    out, kept = oracle.token_topk_decode(q, k, v, case["lens"], topk, local, SINK, oracle.default_scale())
    assert np.array_equal(kept.numpy(), gold["kept"])
    assert np.abs(out.numpy() - gold["out"]).max() < 5e-5
    if name == "ls_tok_fp32":           # lengths at the threshold stay dense, one more token selects
        lens = [int(x) for x in case["lens"]]
        at, over = lens.index(SINK + topk + local), lens.index(SINK + topk + local + 1)
        assert (gold["kept"][at] < 0).all() and (gold["kept"][over] >= 0).all()


def test_view_defaults_equal_plain_oracle():
    case, st, q = case_state("ragged_fp32", seed=2)
    summ = oracle.summaries(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"],
                            st["summary_stride"])
    a, la = oracle.select(q, summ, st["kv_indices"], st["kv_indptr"], case["topk"])
    b, lb, _ = oracle.select_v(q, summ, st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"], case["topk"], 0, 1)
    assert torch.equal(a, b) and torch.equal(la, lb)
