"""The tensor-core prefilter of the bf16 selection against the plain canonical path.

Without a score output the selection kernel scores every page approximately on the tensor cores, keeps the pages
that can still belong to the top-k under a rigorous error bound, and scores only those in the canonical fp32
order; asked for the scores, it scores every page canonically.  Both must pick the same pages in the same order,
bit for bit, whatever the data: ordinary scores, huge and tiny magnitudes, rows of very different scale, heavy
cancellation, exact ties, all-equal rows (the candidate list overflows), infinities.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(q, summ, indices, indptr, last, k, num_pages, view=None):
    from kinetics_b200 import ops
    dev = q.device
    status = ops.new_status(dev)
    B, Hkv = summ.shape[0], summ.shape[1]
    width = k + 1 if view is None else view.row_width(k)
    rows = B if view is None or view.page_count is None else view.page_count.numel()
    la = torch.full((rows, Hkv, width), -7, dtype=torch.int32, device=dev)
    lb = torch.full_like(la, -7)
    scores = torch.zeros(rows, Hkv, summ.shape[2], device=dev)
    a = ops.select_pages(q, summ, indices, indptr, last, k, num_pages, out_logical=la, status=status, view=view)
    b = ops.select_pages(q, summ, indices, indptr, last, k, num_pages, out_logical=lb, out_scores=scores,
                         status=status, view=view)
    ops.raise_on_status(status)
    assert torch.equal(a, b) and torch.equal(la, lb)
    return la


def _table(B, n_pages, dev, seed):
    g = torch.Generator().manual_seed(seed)
    total = B * n_pages
    ids = torch.randperm(total, generator=g).to(torch.int32).to(dev)
    indptr = (torch.arange(B + 1, dtype=torch.int32) * n_pages).to(dev)
    last = torch.randint(1, 17, (B,), generator=g).to(torch.int32).to(dev)
    return ids, indptr, last, total


@pytest.mark.parametrize("G,Hkv,k,n", [(4, 1, 128, 2048), (8, 2, 64, 531), (1, 3, 16, 200), (2, 2, 1024, 1500),
                                       (4, 1, 32, 33)])
def test_prefilter_equals_canonical_on_random_scores(cuda_device, G, Hkv, k, n):
    B = 256
    torch.manual_seed(G * 100 + n)
    summ = torch.randn(B, Hkv, n + 5, 128, device=cuda_device, dtype=torch.bfloat16)
    q = torch.randn(B, Hkv * G, 128, device=cuda_device, dtype=torch.bfloat16)
    ids, indptr, last, total = _table(B, n + 1, cuda_device, 1)
    _both(q, summ, ids, indptr, last, k, total)


@pytest.mark.parametrize("case", ["huge", "tiny", "row_scales", "cancellation", "ties", "all_equal", "infinity",
                                  "zeros"])
def test_prefilter_equals_canonical_on_hostile_data(cuda_device, case):
    B, Hkv, G, k, n = 64, 2, 4, 48, 777
    torch.manual_seed(sum(map(ord, case)))
    summ = torch.randn(B, Hkv, n + 3, 128, device=cuda_device)
    q = torch.randn(B, Hkv * G, 128, device=cuda_device)
    if case == "huge":
        summ *= 3e18; q *= 1e15
    elif case == "tiny":
        summ *= 1e-20; q *= 1e-18
    elif case == "row_scales":
        summ *= torch.logspace(-6, 6, n + 3, device=cuda_device)[torch.randperm(n + 3, device=cuda_device)][None, None, :, None]
    elif case == "cancellation":
        # every row is (x, -x + small): the score is a tiny difference of large terms, all of them near ties
        half = torch.randn(B, Hkv, n + 3, 64, device=cuda_device) * 100
        summ = torch.cat([half, half + torch.randn_like(half) * 1e-2], dim=-1)
        qh = torch.randn(B, Hkv * G, 64, device=cuda_device)
        q = torch.cat([qh, -qh], dim=-1)
    elif case == "ties":
        summ[:, :, 100:400] = summ[:, :, 0:300]            # 300 exact duplicates: ties go to the lower page
    elif case == "all_equal":
        summ[:] = summ[:, :, :1]
    elif case == "infinity":
        summ[::3, :, 17, 5] = float("inf")
        summ[1::3, :, 40, 9] = float("-inf")
    elif case == "zeros":
        summ.zero_()
    summ = summ.to(torch.bfloat16)
    q = q.to(torch.bfloat16)
    ids, indptr, last, total = _table(B, n + 1, cuda_device, 2)
    la = _both(q, summ, ids, indptr, last, k, total)
    if case in ("all_equal", "zeros"):
        assert torch.equal(la[:, :, :k].cpu(), torch.arange(k, dtype=torch.int32).expand(B, Hkv, k))
    if case == "ties":
        # of two duplicate pages the lower one is never missing when the higher one was picked
        picked = torch.zeros(B, Hkv, n + 3, dtype=torch.bool, device=cuda_device).scatter_(2, la[:, :, :k].long(), True)
        assert not (picked[:, :, 100:400] & ~picked[:, :, 0:300]).any()


def test_prefilter_under_a_view_with_ragged_lengths(cuda_device):
    # LiteSys view: sink page in front, local window behind, lists addressed by start + count, summaries by slot
    from kinetics_b200 import ops
    B, Hkv, G, k, slots, stride = 24, 2, 4, 8, 40, 130
    g = torch.Generator().manual_seed(5)
    summ = torch.randn(slots, Hkv, stride, 128, generator=g).to(torch.bfloat16).to(cuda_device)
    q = torch.randn(B, Hkv * G, 128, generator=g).to(torch.bfloat16).to(cuda_device)
    slot = torch.randperm(slots, generator=g)[:B].to(torch.int32)
    lens = torch.randint(3, 16 * (stride - 2), (B,), generator=g)
    lens[0], lens[1], lens[2] = 4 + 16 * (k + 1) + 7, 4 + 16 * 17, 5        # just above the budget, a tile edge, tiny
    count = torch.where(lens > 0, 1 + (torch.clamp(lens - 4, min=0) + 15) // 16, torch.zeros_like(lens)).to(torch.int32)
    last = torch.where(lens > 4, (lens - 4 - 1) % 16 + 1, lens).to(torch.int32)
    start = (slot * stride).to(torch.int32)
    ids = torch.arange(slots * stride, dtype=torch.int32)
    view = ops.PageView(4, 7, count.to(cuda_device), slot.to(cuda_device))
    _both(q, summ, ids.to(cuda_device), start.to(cuda_device), last.to(cuda_device), k, slots * stride, view=view)
