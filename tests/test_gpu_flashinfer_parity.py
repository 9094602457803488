"""The decode kernels against flashinfer's paged batch decode -- the library the reference calls for this
step (benchmark/blocktopk_decoder.py:153-160,176-178,255-265; dense_decoder.py:149-156,168-170).

flashinfer builds its kernel with nvcc on first use; when that is not possible on the machine the
tests are skipped (the oracle tests do not depend on it).
"""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fi_decode(cuda_device, tmp_path_factory):
    os.environ.setdefault("FLASHINFER_WORKSPACE_BASE", str(tmp_path_factory.mktemp("flashinfer")))
    try:
        import flashinfer
        ws = torch.empty(128 * 1024 * 1024, dtype=torch.uint8, device=cuda_device)
        wrapper = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    except Exception as e:                                   # pragma: no cover - depends on the machine
        pytest.skip(f"flashinfer unavailable: {e}")

    def run(q, cache, indices, indptr, last, hq, hkv):
        try:
            wrapper.plan(indptr, indices, last, hq, hkv, 128, 16, pos_encoding_mode="NONE",
                         q_data_type=q.dtype, kv_data_type=cache.dtype)
            return wrapper.run(q, cache)
        except Exception as e:                               # pragma: no cover
            pytest.skip(f"flashinfer could not build or run its decode kernel here: {e}")
    return run


def test_sparse_decode_matches_flashinfer_on_the_selected_pages(cuda_device, fi_decode):
    # the reference's TP=8 shard: 1 KV head, 4 query heads; the selected list is the page table flashinfer gets
    from kinetics_b200 import ops
    B, n, k, G = 64, 256, 32, 4
    torch.manual_seed(21)
    total = B * (n + 1)
    cache = torch.randn(total, 2, 16, 1, 128, device=cuda_device, dtype=torch.bfloat16)
    q = torch.randn(B, G, 128, device=cuda_device, dtype=torch.bfloat16)
    g = torch.Generator(device="cpu").manual_seed(5)
    table = torch.randperm(total, generator=g).to(torch.int32).to(cuda_device)
    indptr = torch.arange(B + 1, dtype=torch.int32, device=cuda_device) * (n + 1)
    last = torch.randint(1, 17, (B,), generator=g).to(torch.int32).to(cuda_device)
    status = ops.new_status(cuda_device)
    summ = torch.zeros(B, 1, n + 1, 128, device=cuda_device, dtype=torch.bfloat16)
    ops.build_summaries(cache, summ, table, indptr, last, status=status)
    sel = ops.select_pages(q, summ, table, indptr, last, k, total, status=status)          # [B, 1, k+1]
    ws = torch.empty(16 << 20, dtype=torch.uint8, device=cuda_device)      # the library's own split policy
    out = ops.sparse_decode(q, cache, sel, indptr, last, workspace=ws, status=status)
    one = ops.sparse_decode(q, cache, sel, indptr, last, num_splits=1, status=status)
    ops.raise_on_status(status)
    sel_indptr = torch.arange(B + 1, dtype=torch.int32, device=cuda_device) * (k + 1)
    ref = fi_decode(q, cache, sel.view(-1).contiguous(), sel_indptr, last, G, 1)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(one.float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_dense_decode_matches_flashinfer(cuda_device, fi_decode):
    from kinetics_b200 import ops
    B, Hkv, G = 32, 2, 4
    torch.manual_seed(22)
    g = torch.Generator(device="cpu").manual_seed(6)
    counts = torch.randint(1, 200, (B,), generator=g)
    indptr_c = torch.zeros(B + 1, dtype=torch.int64)
    indptr_c[1:] = torch.cumsum(counts, 0)
    total = int(indptr_c[-1])
    cache = torch.randn(total + 3, 2, 16, Hkv, 128, device=cuda_device, dtype=torch.bfloat16)
    q = torch.randn(B, Hkv * G, 128, device=cuda_device, dtype=torch.bfloat16)
    table = torch.randperm(total + 3, generator=g)[:total].to(torch.int32).to(cuda_device)
    indptr = indptr_c.to(torch.int32).to(cuda_device)
    last = torch.randint(1, 17, (B,), generator=g).to(torch.int32).to(cuda_device)
    status = ops.new_status(cuda_device)
    ws = torch.empty(16 << 20, dtype=torch.uint8, device=cuda_device)
    out = ops.dense_decode(q, cache, table, indptr, last, int(counts.max()), workspace=ws, status=status)
    ops.raise_on_status(status)
    ref = fi_decode(q, cache, table, indptr, last, Hkv * G, Hkv)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
