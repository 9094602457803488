"""CUDA kernels (through the C ABI) against the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest
import torch

from helpers import CASES, LITESYS_CASES, P, SINK, case_state, load_golden, paged_state, random_case, to_dev
from oracle import oracle

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32)


def _ops():
    from kinetics_b200 import ops
    return ops


def _tol(dtype):
    # north-star tolerances: 1e-4 abs/rel in fp32, 2e-2 in bf16
    return 1e-4 if dtype == torch.float32 else 2e-2


# ---------------------------------------------------------------- append + summaries

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_append_and_summaries_bit_exact(cuda_device, dtype):
    ops = _ops()
    torch.manual_seed(7)
    B, Hkv, npg_max, steps = 5, 2, 4, 50
    total = B * npg_max + 3
    table = torch.randperm(total)[: B * npg_max].view(B, npg_max).to(torch.int32)
    cache_c = torch.zeros(total, 2, P, Hkv, 128, dtype=dtype)
    summ_c = torch.zeros(B, Hkv, npg_max, 128, dtype=dtype)
    cache_g, summ_g = cache_c.to(cuda_device), summ_c.to(cuda_device)
    status = ops.new_status(cuda_device)
    for s in range(steps):
        npg = s // P + 1
        indices = table[:, :npg].contiguous().view(-1)
        indptr = (torch.arange(B + 1) * npg).to(torch.int32)
        last = torch.full((B,), s % P + 1, dtype=torch.int32)
        k = torch.randn(B, Hkv, 128).to(dtype)
        v = torch.randn(B, Hkv, 128).to(dtype)
        oracle.append(k, v, cache_c, summ_c, indices, indptr, last)
        ops.append_kv(k.to(cuda_device), v.to(cuda_device), cache_g, summ_g, indices.to(cuda_device),
                      indptr.to(cuda_device), last.to(cuda_device), status=status)
    ops.raise_on_status(status)
    assert torch.equal(_bits(cache_g.cpu()), _bits(cache_c))
    assert torch.equal(_bits(summ_g.cpu()), _bits(summ_c))
    # bulk rebuild gives the same summaries
    rebuilt = torch.zeros_like(summ_g)
    ops.build_summaries(cache_g, rebuilt, indices.to(cuda_device), indptr.to(cuda_device), last.to(cuda_device),
                        status=status)
    ops.raise_on_status(status)
    assert torch.equal(_bits(rebuilt.cpu()), _bits(summ_c))


def test_append_ragged_and_empty(cuda_device):
    ops = _ops()
    dtype = torch.bfloat16
    lens = [0, 17, 1, 32]                      # an empty slot, mid-page, first token, page just filled
    q, k, v = random_case(3, 4, 2, 2, lens, dtype)
    st = paged_state(k, v, lens, dtype, seed=1, fill=0.0)
    # drop the newest token from the cache, append it back with the kernel
    want = st["kv_cache"].clone()
    cache = st["kv_cache"].clone()
    knew = torch.zeros(4, 2, 128, dtype=dtype)
    vnew = torch.zeros(4, 2, 128, dtype=dtype)
    for b, n in enumerate(lens):
        if n == 0:
            continue
        page = int(st["kv_indices"][st["kv_indptr"][b + 1] - 1])
        slot = int(st["kv_last_page_len"][b]) - 1
        knew[b], vnew[b] = cache[page, 0, slot], cache[page, 1, slot]
        cache[page, :, slot] = 0
    summ = torch.zeros(4, 2, st["summary_stride"], 128, dtype=dtype)
    d = to_dev(st, cuda_device)
    cache_g, summ_g = cache.to(cuda_device), summ.to(cuda_device)
    status = ops.new_status(cuda_device)
    ops.append_kv(knew.to(cuda_device), vnew.to(cuda_device), cache_g, summ_g, d["kv_indices"], d["kv_indptr"],
                  d["kv_last_page_len"], status=status)
    ops.raise_on_status(status)
    assert torch.equal(_bits(cache_g.cpu()), _bits(want))
    ref = oracle.summaries(want, st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"], st["summary_stride"])
    for b, n in enumerate(lens):
        if n:
            lastp = st["npages"][b] - 1
            assert torch.equal(_bits(summ_g.cpu()[b, :, lastp]), _bits(ref[b, :, lastp]))


# ---------------------------------------------------------------- selection

def _select_both(ops, q, st, topk, device, view=None):
    summ = oracle.summaries(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"],
                            st["summary_stride"])
    sc = oracle.scores(q, summ, st["kv_indptr"])
    phys, logical = oracle.select_from_scores(sc, st["kv_indices"], st["kv_indptr"], topk)
    d = to_dev(st, device)
    summ_g = torch.zeros_like(summ, device=device)
    status = ops.new_status(device)
    ops.build_summaries(d["kv_cache"], summ_g, d["kv_indices"], d["kv_indptr"], d["kv_last_page_len"], status=status)
    assert torch.equal(_bits(summ_g.cpu()), _bits(summ))
    B, Hkv = summ.shape[:2]
    out_l = torch.empty(B, Hkv, topk + 1, dtype=torch.int32, device=device)
    out_s = torch.full((B, Hkv, st["summary_stride"]), float("nan"), device=device)
    out_p = ops.select_pages(q.to(device), summ_g, d["kv_indices"], d["kv_indptr"], d["kv_last_page_len"], topk,
                             st["num_pages"], out_logical=out_l, out_scores=out_s, status=status, view=view)
    ops.raise_on_status(status)
    return (phys, logical, sc), (out_p.cpu(), out_l.cpu(), out_s.cpu()), d, summ_g


@pytest.mark.parametrize("name", sorted(CASES))
def test_select_bit_exact_on_golden_cases(cuda_device, name):
    ops = _ops()
    case, st, q = case_state(name, seed=4)
    (phys, logical, sc), (gp, gl, gs), _, _ = _select_both(ops, q, st, case["topk"], cuda_device)
    assert torch.equal(gl, logical)
    assert torch.equal(gp, phys)
    for b, npg in enumerate(st["npages"]):
        assert torch.equal(gs[b, :, : npg - 1].view(torch.int32), sc[b, :, : npg - 1].view(torch.int32))
    # and the reference's own kept sets
    gold = load_golden(name)
    for b, npg in enumerate(st["npages"]):
        cnt = min(case["topk"], npg - 1)
        for h in range(gl.shape[1]):
            ref = gold["kept"][b, h][gold["kept"][b, h] >= 0]
            assert np.array_equal(np.sort(gl[b, h, :cnt].numpy()), ref)


@pytest.mark.parametrize("dtype,G,Hkv,topk,lens", [
    (torch.bfloat16, 4, 1, 128, [32769, 32768, 20000]),      # 2048 scored pages, the headline shape
    (torch.bfloat16, 8, 2, 64, [16385, 1025, 4000, 9999]),
    (torch.float32, 4, 1, 16, [2049, 2049]),
    (torch.bfloat16, 2, 3, 32, [513, 1, 16, 17, 5000]),
    (torch.float32, 1, 2, 1, [100, 33]),
    (torch.bfloat16, 4, 1, 1024, [20001]),                   # largest budget
])
def test_select_bit_exact_random(cuda_device, dtype, G, Hkv, topk, lens):
    ops = _ops()
    q, k, v = random_case(99, len(lens), Hkv, G, lens, dtype)
    st = paged_state(k, v, lens, dtype, seed=8)
    (phys, logical, sc), (gp, gl, gs), _, _ = _select_both(ops, q, st, topk, cuda_device)
    assert torch.equal(gl, logical)
    assert torch.equal(gp, phys)


@pytest.mark.parametrize("order", [None, "longest_first", "shuffled"])
def test_select_many_ragged_items_per_cta(cuda_device, order):
    """More (sequence, kv head) items than resident CTAs: every CTA streams several items of different lengths
    back to back through its ring (the stage <-> warp assignment carries over from item to item), some of them
    empty or shorter than the budget.  With a sequence order in the view the CTAs take the sequences in that
    order, every other round reversed; the rows written must not depend on it."""
    ops = _ops()
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(77)
    lens = torch.randint(17, 3000, (470,), generator=g).tolist()
    lens[5], lens[6], lens[100], lens[469] = 1, 16, 0, 16 * 24 + 1
    q, k, v = random_case(12, len(lens), 2, 2, lens, dtype)
    st = paged_state(k, v, lens, dtype, seed=21)
    view = None
    if order is not None:
        perm = torch.argsort(torch.tensor(lens), descending=True, stable=True) if order == "longest_first" \
            else torch.randperm(len(lens), generator=g)
        view = ops.PageView(0, 1, None, None, perm.to(torch.int32).to(cuda_device))
    (phys, logical, sc), (gp, gl, gs), _, _ = _select_both(ops, q, st, 24, cuda_device, view=view)
    assert torch.equal(gl, logical)
    assert torch.equal(gp, phys)


def test_select_reports_an_order_entry_that_is_no_sequence(cuda_device):
    ops = _ops()
    lens = [100, 200, 300]
    q, k, v = random_case(3, 3, 1, 2, lens, torch.bfloat16)
    st = to_dev(paged_state(k, v, lens, torch.bfloat16, seed=2), cuda_device)
    summ = torch.zeros(3, 1, st["summary_stride"], 128, device=cuda_device, dtype=torch.bfloat16)
    status = ops.new_status(cuda_device)
    ops.build_summaries(st["kv_cache"], summ, st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"], status=status)
    view = ops.PageView(0, 1, None, None, torch.tensor([2, 7, 0], dtype=torch.int32, device=cuda_device))
    ops.select_pages(q.to(cuda_device), summ, st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"], 4,
                     st["num_pages"], status=status, view=view)
    with pytest.raises(RuntimeError):
        ops.raise_on_status(status)


def test_select_ties_go_to_lowest_page(cuda_device):
    ops = _ops()
    dtype = torch.bfloat16
    lens = [16 * 300 + 3, 16 * 40 + 16]
    q, k, v = random_case(5, 2, 2, 4, lens, dtype)
    k[0] = 0.0                                   # all scores equal (+0)
    k[1, :, : 16 * 20] = k[1, :, 16 * 20: 16 * 40]   # every score appears twice
    st = paged_state(k, v, lens, dtype, seed=3)
    (phys, logical, sc), (gp, gl, gs), _, _ = _select_both(ops, q, st, 24, cuda_device)
    assert gl[0, 0, :24].tolist() == list(range(24))
    assert torch.equal(gl, logical) and torch.equal(gp, phys)


def test_select_reports_bad_page_id(cuda_device):
    ops = _ops()
    dtype = torch.float32
    lens = [200]
    q, k, v = random_case(6, 1, 1, 4, lens, dtype)
    st = paged_state(k, v, lens, dtype, seed=3)
    d = to_dev(st, cuda_device)
    summ = oracle.summaries(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"],
                            st["summary_stride"]).to(cuda_device)
    bad = d["kv_indices"].clone()
    bad[:] = st["num_pages"] + 5
    status = ops.new_status(cuda_device)
    ops.select_pages(q.to(cuda_device), summ, bad, d["kv_indptr"], d["kv_last_page_len"], 4, st["num_pages"],
                     status=status)
    assert int(status.item()) == 1
    # the decode kernel skips such pages instead of reading them
    sel = torch.full((1, 1, 5), st["num_pages"] + 5, dtype=torch.int32, device=cuda_device)
    status.zero_()
    out = ops.sparse_decode(q.to(cuda_device), d["kv_cache"], sel, d["kv_indptr"], d["kv_last_page_len"],
                            num_splits=1, variant=1, status=status)
    assert int(status.item()) == 1
    assert torch.isfinite(out).all()


def test_tensor_core_decode_skips_bad_pages(cuda_device):
    ops = _ops()
    dtype = torch.bfloat16
    lens = [200, 90]
    q, k, v = random_case(6, 2, 2, 4, lens, dtype)
    st = paged_state(k, v, lens, dtype, seed=3)
    d = to_dev(st, cuda_device)
    # a list whose middle entries are out of range: they are skipped, the rest is attended
    good = oracle.select(q, oracle.summaries(st["kv_cache"], st["kv_indices"], st["kv_indptr"],
                                             st["kv_last_page_len"], st["summary_stride"]),
                         st["kv_indices"], st["kv_indptr"], 6)[0]
    bad = good.clone()
    bad[:, :, 2] = st["num_pages"] + 9
    bad[:, :, 3] = -4
    status = ops.new_status(cuda_device)
    out = ops.sparse_decode(q.to(cuda_device), d["kv_cache"], bad.to(cuda_device), d["kv_indptr"],
                            d["kv_last_page_len"], num_splits=1, variant=2, status=status)
    assert int(status.item()) == 1
    ref = ops.sparse_decode(q.to(cuda_device), d["kv_cache"], bad.to(cuda_device), d["kv_indptr"],
                            d["kv_last_page_len"], num_splits=1, variant=1)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


# ---------------------------------------------------------------- decode

VARIANTS = {torch.float32: [1], torch.bfloat16: [1, 2]}   # 1 = fp32 FMA kernel, 2 = tensor-core kernel


def _splits(base, variant):
    """Per-list split counts, plus the balanced partition (-1) where it exists: the tensor-core kernels.
    These cases are small, so the balanced grid is one CTA per 16 page positions and most lists are cut."""
    return tuple(base) + ((-1,) if variant == 2 else ())


@pytest.mark.parametrize("name", sorted(CASES))
def test_sparse_decode_on_golden_cases(cuda_device, name):
    ops = _ops()
    case, st, q = case_state(name, seed=4)
    dtype = q.dtype
    topk = case["topk"]
    (phys, logical, sc), (gp, gl, gs), d, _ = _select_both(ops, q, st, topk, cuda_device)
    ref = oracle.decode(q, st["kv_cache"], phys, topk, st["kv_indptr"], st["kv_last_page_len"],
                        oracle.default_scale())
    gold = load_golden(name)
    tol = _tol(dtype)
    B, Hq = q.shape[:2]
    for variant in VARIANTS[dtype]:
        for splits in _splits((1, 2, 5), variant):
            ws = torch.empty(max(ops.decode_workspace_bytes(B, gp.shape[1], Hq // gp.shape[1], splits), 1),
                             dtype=torch.uint8, device=cuda_device)
            out = ops.sparse_decode(q.to(cuda_device), d["kv_cache"], gp.to(cuda_device), d["kv_indptr"],
                                    d["kv_last_page_len"], workspace=ws, num_splits=splits, variant=variant)
            np.testing.assert_allclose(out.float().cpu().numpy(), ref.numpy(), rtol=tol, atol=tol)
            np.testing.assert_allclose(out.float().cpu().numpy(), gold["out"], rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype,G,Hkv,lens", [
    (torch.bfloat16, 4, 1, [2049, 100, 16, 1]),
    (torch.bfloat16, 8, 2, [777, 1300]),
    (torch.float32, 4, 2, [300, 45]),
    (torch.float32, 1, 1, [64, 65]),
    (torch.bfloat16, 2, 4, [31, 32, 33]),
    (torch.bfloat16, 4, 2, [40, 0, 17, 0]),              # sequences without pages: zero rows
    (torch.bfloat16, 8, 1, [0, 0, 5000, 3, 0, 700]),     # one long list among short ones: cut many times
    (torch.float32, 2, 2, [0, 33, 0]),
])
def test_dense_decode_vs_oracle(cuda_device, dtype, G, Hkv, lens):
    ops = _ops()
    q, k, v = random_case(21, len(lens), Hkv, G, lens, dtype)
    st = paged_state(k, v, lens, dtype, seed=9)
    d = to_dev(st, cuda_device)
    ref = oracle.decode(q, st["kv_cache"], st["kv_indices"], -1, st["kv_indptr"], st["kv_last_page_len"],
                        oracle.default_scale())
    tol = _tol(dtype)
    B, Hq = q.shape[:2]
    for variant in VARIANTS[dtype]:
        for splits in (1, 3, 0):
            s_eff = splits or ops.decode_num_splits(B, Hkv, G, max(st["npages"]), dtype)
            ws = torch.empty(max(ops.decode_workspace_bytes(B, Hkv, G, s_eff), 1), dtype=torch.uint8,
                             device=cuda_device)
            out = ops.dense_decode(q.to(cuda_device), d["kv_cache"], d["kv_indices"], d["kv_indptr"],
                                   d["kv_last_page_len"], max(st["npages"]), workspace=ws, num_splits=splits,
                                   variant=variant)
            np.testing.assert_allclose(out.float().cpu().numpy(), ref.numpy(), rtol=tol, atol=tol)


def test_sparse_equals_dense_when_budget_covers_everything(cuda_device):
    ops = _ops()
    dtype = torch.bfloat16
    lens = [500, 129]
    q, k, v = random_case(22, 2, 2, 4, lens, dtype)
    st = paged_state(k, v, lens, dtype, seed=9)
    (phys, *_), (gp, *_), d, _ = _select_both(ops, q, st, 40, cuda_device)
    for variant in (1, 2):
        a = ops.sparse_decode(q.to(cuda_device), d["kv_cache"], gp.to(cuda_device), d["kv_indptr"],
                              d["kv_last_page_len"], num_splits=1, variant=variant)
        b = ops.dense_decode(q.to(cuda_device), d["kv_cache"], d["kv_indices"], d["kv_indptr"],
                             d["kv_last_page_len"], max(st["npages"]), num_splits=1, variant=variant)
        assert torch.equal(a, b)


def test_large_logits_do_not_overflow(cuda_device):
    ops = _ops()
    dtype = torch.bfloat16
    lens = [400]
    q, k, v = random_case(23, 1, 1, 4, lens, dtype, scale=6.0)   # logits of a few hundred
    st = paged_state(k, v, lens, dtype, seed=9)
    d = to_dev(st, cuda_device)
    ref = oracle.decode(q, st["kv_cache"], st["kv_indices"], -1, st["kv_indptr"], st["kv_last_page_len"],
                        oracle.default_scale())
    for variant in (1, 2):
        out = ops.dense_decode(q.to(cuda_device), d["kv_cache"], d["kv_indices"], d["kv_indptr"],
                               d["kv_last_page_len"], 25, num_splits=1, variant=variant)
        assert torch.isfinite(out).all()
        np.testing.assert_allclose(out.float().cpu().numpy(), ref.numpy(), rtol=3e-2, atol=3e-2)


# ---------------------------------------------------------------- page views (LiteSys semantics)

def _view_roundtrip(ops, device, q, st, topk, sink, local, gold_out=None, scattered=False):
    """build summaries, select and decode under a view on the GPU; compare with the oracle under the same view"""
    dtype = q.dtype
    B, Hq = q.shape[:2]
    Hkv = st["kv_cache"].shape[3]
    summ = oracle.summaries_v(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"],
                              st["summary_stride"], sink)
    phys, logical, sc = oracle.select_v(q, summ, st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"], topk,
                                        sink, local)
    ref = oracle.decode_v(q, st["kv_cache"], phys, topk, st["kv_indptr"], st["kv_last_page_len"],
                          oracle.default_scale(), sink, local)
    ref_dense = oracle.decode_v(q, st["kv_cache"], st["kv_indices"], -1, st["kv_indptr"], st["kv_last_page_len"],
                                oracle.default_scale(), sink, local)
    d = to_dev(st, device)
    indptr, rows = d["kv_indptr"], B
    page_count = slot_index = None
    if scattered:
        # lists given by (start, count), summaries kept in other rows than the batch order
        page_count = (d["kv_indptr"][1:] - d["kv_indptr"][:-1]).contiguous()
        indptr = d["kv_indptr"][:-1].contiguous()
        perm = torch.randperm(B + 3, generator=torch.Generator().manual_seed(5))[:B]
        slot_index = perm.to(torch.int32).to(device)
        rows = B + 3
    view = ops.PageView(sink, local, page_count, slot_index)
    summ_g = torch.zeros(rows, Hkv, st["summary_stride"], 128, dtype=dtype, device=device)
    status = ops.new_status(device)
    ops.build_summaries(d["kv_cache"], summ_g, d["kv_indices"], indptr, d["kv_last_page_len"], status=status,
                        view=view)
    got_summ = summ_g.cpu() if slot_index is None else summ_g.cpu()[slot_index.cpu().long()]
    for b, npg in enumerate(st["npages"]):
        assert torch.equal(_bits(got_summ[b, :, :npg]), _bits(summ[b, :, :npg]))
    width = view.row_width(topk)
    assert width == phys.shape[-1]
    out_l = torch.empty(B, Hkv, width, dtype=torch.int32, device=device)
    sel = ops.select_pages(q.to(device), summ_g, d["kv_indices"], indptr, d["kv_last_page_len"], topk,
                           st["num_pages"], out_logical=out_l, status=status, view=view)
    ops.raise_on_status(status)
    assert torch.equal(out_l.cpu(), logical)
    assert torch.equal(sel.cpu(), phys)
    tol = _tol(dtype)
    for variant in VARIANTS[dtype]:
        for splits in _splits((1, 3), variant):
            ws = torch.empty(max(ops.decode_workspace_bytes(B, Hkv, Hq // Hkv, splits), 1), dtype=torch.uint8,
                             device=device)
            out = ops.sparse_decode(q.to(device), d["kv_cache"], sel, indptr, d["kv_last_page_len"], workspace=ws,
                                    num_splits=splits, variant=variant, view=view, topk=topk, status=status)
            np.testing.assert_allclose(out.float().cpu().numpy(), ref.numpy(), rtol=tol, atol=tol)
            if gold_out is not None:
                np.testing.assert_allclose(out.float().cpu().numpy(), gold_out, rtol=tol, atol=tol)
            dn = ops.dense_decode(q.to(device), d["kv_cache"], d["kv_indices"], indptr, d["kv_last_page_len"],
                                  max(st["npages"]), workspace=ws, num_splits=splits, variant=variant, view=view,
                                  status=status)
            np.testing.assert_allclose(dn.float().cpu().numpy(), ref_dense.numpy(), rtol=tol, atol=tol)
    ops.raise_on_status(status)


@pytest.mark.parametrize("scattered", [False, True])
@pytest.mark.parametrize("name", sorted(LITESYS_CASES))
def test_view_kernels_on_litesys_golden_cases(cuda_device, name, scattered):
    ops = _ops()
    case, st, q = case_state(name, seed=6)
    gold = load_golden(name)
    _view_roundtrip(ops, cuda_device, q, st, case["topk"], SINK, case["local"], gold_out=gold["out"],
                    scattered=scattered)


@pytest.mark.parametrize("dtype,G,Hkv,topk,sink,local,lens", [
    (torch.bfloat16, 8, 1, 32, 4, 100, [5000, 3, 4, 5, 20, 21, 1234]),
    (torch.bfloat16, 4, 2, 16, 4, 0, [4 + 16 * 40, 4 + 16 * 17 + 1, 4 + 16 * 16]),     # lengths that end on a block edge
    (torch.float32, 2, 2, 8, 7, 33, [700, 8, 300]),
    (torch.bfloat16, 4, 1, 64, 0, 50, [2049, 100]),                                 # no sink, wider always-kept tail
])
def test_view_kernels_random(cuda_device, dtype, G, Hkv, topk, sink, local, lens):
    ops = _ops()
    q, k, v = random_case(31, len(lens), Hkv, G, lens, dtype)
    st = paged_state(k, v, lens, dtype, seed=10, sink=sink)
    _view_roundtrip(ops, cuda_device, q, st, topk, sink, local)


def test_view_append_maintains_block_summaries(cuda_device):
    # tokens appended one at a time through the sink page and the pages behind it
    ops = _ops()
    dtype = torch.bfloat16
    B, Hkv, sink, steps = 3, 2, 4, 41
    per = 1 + (steps - sink + P - 1) // P
    total = B * per + 2
    table = torch.randperm(total, generator=torch.Generator().manual_seed(3))[: B * per].view(B, per).to(torch.int32)
    cache = torch.zeros(total, 2, P, Hkv, 128, dtype=dtype, device=cuda_device)
    summ = torch.zeros(B, Hkv, per, 128, dtype=dtype, device=cuda_device)
    view = ops.PageView(sink, 0)
    ks, vs = [], []
    status = ops.new_status(cuda_device)
    for s_ in range(steps):
        n = s_ + 1
        npg = 1 if n <= sink else 1 + (n - sink + P - 1) // P
        last = n if n <= sink else (n - sink - 1) % P + 1
        indices = table[:, :npg].contiguous().view(-1).to(cuda_device)
        indptr = (torch.arange(B + 1) * npg).to(torch.int32).to(cuda_device)
        lastt = torch.full((B,), last, dtype=torch.int32, device=cuda_device)
        k = torch.randn(B, Hkv, 128).to(dtype)
        v = torch.randn(B, Hkv, 128).to(dtype)
        ks.append(k); vs.append(v)
        ops.append_kv(k.to(cuda_device), v.to(cuda_device), cache, summ, indices, indptr, lastt, status=status,
                      view=view)
    ops.raise_on_status(status)
    kk = torch.stack(ks, 2).float()            # [B, Hkv, steps, D]
    vv = torch.stack(vs, 2).float()
    st = paged_state(kk, vv, [steps] * B, dtype, seed=0, sink=sink, summary_stride=per)
    want = oracle.summaries_v(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"], per, sink)
    assert torch.equal(_bits(summ.cpu()), _bits(want))


# ---------------------------------------------------------------- small ops

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [128, 4096, 1000])
def test_rmsnorm(cuda_device, dtype, cols):
    ops = _ops()
    torch.manual_seed(1)
    x = torch.randn(37, cols).to(dtype)
    w = (torch.rand(cols) + 0.5).to(dtype)
    ref = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float())
    out = ops.rmsnorm(x.to(cuda_device), w.to(cuda_device), 1e-6)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(out.float().cpu(), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(cuda_device, dtype):
    ops = _ops()
    torch.manual_seed(2)
    g, u = torch.randn(3, 1, 1536).to(dtype), torch.randn(3, 1, 1536).to(dtype)
    ref = torch.nn.functional.silu(g.float()) * u.float()
    out = ops.silu_mul(g.to(cuda_device), u.to(cuda_device))
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(out.float().cpu(), ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul_on_the_halves_of_one_gemm_output(cuda_device, dtype):
    """gate and up as the two halves of a [rows, 2 * cols] tensor give the bits of the contiguous call."""
    ops = _ops()
    torch.manual_seed(3)
    gu = torch.randn(37, 2 * 768).to(dtype).to(cuda_device)
    g, u = gu[:, :768], gu[:, 768:]
    out = ops.silu_mul(g, u)
    ref = ops.silu_mul(g.contiguous(), u.contiguous())
    assert out.is_contiguous() and torch.equal(_bits(out.cpu()), _bits(ref.cpu()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [512, 4096, 5120])
def test_add_rmsnorm(cuda_device, dtype, cols):
    ops = _ops()
    torch.manual_seed(3)
    x, r = torch.randn(19, cols).to(dtype), torch.randn(19, cols).to(dtype)
    w = (torch.rand(cols) + 0.5).to(dtype)
    s_ref = (x.float() + r.float()).to(dtype)
    n_ref = s_ref.float() * torch.rsqrt(s_ref.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    s, n = ops.add_rmsnorm(x.to(cuda_device), r.to(cuda_device), w.to(cuda_device), 1e-6)
    assert torch.equal(s.cpu(), s_ref)                       # the stored sum is the rounded sum
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(n.float().cpu(), n_ref, rtol=tol, atol=tol)
    s0, n0 = ops.add_rmsnorm(x.to(cuda_device), None, w.to(cuda_device), 1e-6)
    n0_ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    torch.testing.assert_close(n0.float().cpu(), n0_ref, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qkv_norm_split(cuda_device, dtype):
    ops = _ops()
    torch.manual_seed(4)
    B, Hq, Hkv = 7, 8, 2
    proj = torch.randn(B, (Hq + 2 * Hkv) * 128).to(dtype)
    wq, wk = (torch.rand(128) + 0.5).to(dtype), (torch.rand(128) + 0.5).to(dtype)
    q, k, v = ops.qkv_norm(proj.to(cuda_device), wq.to(cuda_device), wk.to(cuda_device), 1e-6, Hq, Hkv)

    def norm(t, w):
        t = t.float()
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()

    pq, pk, pv = proj.split((Hq * 128, Hkv * 128, Hkv * 128), dim=-1)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(q.float().cpu(), norm(pq.view(B, Hq, 128), wq), rtol=tol, atol=tol)
    torch.testing.assert_close(k.float().cpu(), norm(pk.view(B, Hkv, 128), wk), rtol=tol, atol=tol)
    assert torch.equal(v.cpu(), pv.reshape(B, Hkv, 128))


@pytest.mark.parametrize("sink", [0, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_append_tokens_chunks_bit_exact(cuda_device, dtype, sink):
    # ragged chunks appended behind ragged prefixes: cache and the touched summaries follow the oracle
    ops = _ops()
    before = [0, 37, 5, 100, 16]
    chunk = [50, 1, 0, 29, 16]
    after = [a + c for a, c in zip(before, chunk)]
    B, Hkv = len(before), 2
    q, k, v = random_case(41, B, Hkv, 1, after, dtype)
    st_after = paged_state(k, v, after, dtype, seed=2, sink=sink, fill=0.0)
    # the same table, holding only the prefix
    cache = st_after["kv_cache"].clone()
    kk = torch.cat([k[b, :, before[b]:after[b]].transpose(0, 1) for b in range(B)]).to(dtype).contiguous()
    vv = torch.cat([v[b, :, before[b]:after[b]].transpose(0, 1) for b in range(B)]).to(dtype).contiguous()
    ai = torch.tensor([0] + list(np.cumsum(chunk)), dtype=torch.int32)
    blank = torch.zeros_like(kk)
    oracle.append_tokens(blank, blank, ai, cache, st_after["kv_indices"], st_after["kv_indptr"],
                         st_after["kv_last_page_len"], sink)                      # wipe the chunk
    want_cache = cache.clone()
    oracle.append_tokens(kk, vv, ai, want_cache, st_after["kv_indices"], st_after["kv_indptr"],
                         st_after["kv_last_page_len"], sink)
    assert torch.equal(_bits(want_cache), _bits(st_after["kv_cache"]))
    d = to_dev(st_after, cuda_device)
    cache_g = cache.to(cuda_device)
    summ_g = torch.zeros(B, Hkv, st_after["summary_stride"], 128, dtype=dtype, device=cuda_device)
    status = ops.new_status(cuda_device)
    view = ops.PageView(sink, 1) if sink else None
    ops.append_tokens(kk.to(cuda_device), vv.to(cuda_device), ai.to(cuda_device), cache_g, summ_g, d["kv_indices"],
                      d["kv_indptr"], d["kv_last_page_len"], status=status, view=view)
    ops.raise_on_status(status)
    assert torch.equal(_bits(cache_g.cpu()), _bits(want_cache))
    want_summ = oracle.summaries_v(want_cache, st_after["kv_indices"], st_after["kv_indptr"],
                                   st_after["kv_last_page_len"], st_after["summary_stride"], sink)

    def page_of(pos):
        return pos // P if sink == 0 else (0 if pos < sink else 1 + (pos - sink) // P)

    got = summ_g.cpu()
    for b in range(B):
        if chunk[b] == 0:
            assert not got[b].any()                      # untouched sequence: nothing rewritten
            continue
        first = page_of(before[b])
        npg = st_after["npages"][b]
        assert torch.equal(_bits(got[b, :, first:npg]), _bits(want_summ[b, :, first:npg]))
        assert not got[b, :, :first].any()               # pages in front of the chunk keep their summaries
