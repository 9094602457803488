"""Property tests of the CPU oracle (hypothesis): what must hold for any paged state."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from helpers import paged_state
from oracle import oracle


@st.composite
def states(draw):
    hkv = draw(st.sampled_from([1, 2]))
    g = draw(st.sampled_from([1, 2, 4]))
    lens = draw(st.lists(st.integers(1, 200), min_size=1, max_size=3))
    topk = draw(st.integers(1, 6))
    sink = draw(st.sampled_from([0, 4]))
    local = draw(st.sampled_from([0, 1, 9, 40])) if sink else 1
    seed = draw(st.integers(0, 10_000))
    return hkv, g, lens, topk, sink, local, seed


def _make(hkv, g, lens, sink, seed, table_seed):
    gen = torch.Generator().manual_seed(seed)
    L = max(lens)
    q = torch.randn(len(lens), hkv * g, 128, generator=gen)
    k = torch.randn(len(lens), hkv, L, 128, generator=gen)
    v = torch.randn(len(lens), hkv, L, 128, generator=gen)
    return q, paged_state(k, v, lens, torch.float32, seed=table_seed, sink=sink)


def _pipeline(q, s, topk, sink, local):
    summ = oracle.summaries_v(s["kv_cache"], s["kv_indices"], s["kv_indptr"], s["kv_last_page_len"],
                              s["summary_stride"], sink)
    phys, logical, _ = oracle.select_v(q, summ, s["kv_indices"], s["kv_indptr"], s["kv_last_page_len"], topk, sink,
                                       local)
    out = oracle.decode_v(q, s["kv_cache"], phys, topk, s["kv_indptr"], s["kv_last_page_len"],
                          oracle.default_scale(), sink, local)
    return phys, logical, out


@settings(max_examples=25, deadline=None)
@given(states())
def test_physical_placement_does_not_matter(p):
    hkv, g, lens, topk, sink, local, seed = p
    q, a = _make(hkv, g, lens, sink, seed, table_seed=1)
    _, b = _make(hkv, g, lens, sink, seed, table_seed=2)        # same tokens, other physical pages
    pa, la, oa = _pipeline(q, a, topk, sink, local)
    pb, lb, ob = _pipeline(q, b, topk, sink, local)
    assert torch.equal(la, lb)
    assert torch.equal(oa, ob)
    # physical ids are the table's entries for the logical picks
    for bi in range(len(lens)):
        tab = a["kv_indices"][a["kv_indptr"][bi]:a["kv_indptr"][bi + 1]]
        row = la[bi, 0]
        assert torch.equal(pa[bi, 0][row >= 0], tab[row[row >= 0].long()])


@settings(max_examples=25, deadline=None)
@given(states())
def test_a_budget_that_covers_everything_is_dense(p):
    hkv, g, lens, _, sink, local, seed = p
    q, s = _make(hkv, g, lens, sink, seed, table_seed=3)
    _, logical, out = _pipeline(q, s, 64, sink, local)
    dense = oracle.decode_v(q, s["kv_cache"], s["kv_indices"], -1, s["kv_indptr"], s["kv_last_page_len"],
                            oracle.default_scale(), sink, local)
    assert torch.equal(out, dense)
    for bi, n in enumerate(s["npages"]):
        assert logical[bi, 0, :n].tolist() == list(range(n))


@settings(max_examples=25, deadline=None)
@given(states())
def test_rows_are_sink_then_picks_then_tail_without_repeats(p):
    hkv, g, lens, topk, sink, local, seed = p
    q, s = _make(hkv, g, lens, sink, seed, table_seed=4)
    _, logical, out = _pipeline(q, s, topk, sink, local)
    assert torch.isfinite(out).all()
    for bi, n in enumerate(s["npages"]):
        for h in range(hkv):
            row = logical[bi, h][logical[bi, h] >= 0].tolist()
            assert len(set(row)) == len(row)
            if local >= 1:
                assert row[-1] == n - 1                   # the newest token's page is always attended
            if sink:
                assert row[0] == 0
