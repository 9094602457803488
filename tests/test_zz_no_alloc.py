"""The allocation-free split decode (ktk_sparse_decode_noalloc) against ktk_sparse_decode.

Some hosts of the library cannot give it a workspace and must not see it allocate (an engine
that handed all device memory to its own page pool at start-up; a decode loop that cannot take
the device-wide synchronisation of an allocation).  For them the split partials live in a fixed
16 MiB array inside the library.  This file calls that entry point through the C ABI, twice in
a row with different inputs and split counts, and expects the very same bits as the entry point
that takes a caller-owned workspace: both run the same kernels over the same split partition,
only the address of the partials differs.  The second call also shows that what the first call
left in the shared array does not leak into later results.

Collected last on purpose (file name), so that a run stopping at the first failure has already
run every other test.
"""
import ctypes

import pytest
import torch

from helpers import paged_state, random_case, to_dev


def _lib():
    from kinetics_b200 import _lib
    return _lib


def _shape(B, Hkv, G, num_pages, dtype_code=1):
    return _lib().Shape(B, Hkv, G, 128, 16, dtype_code, num_pages)


def test_request_beyond_the_built_in_array_is_refused_on_the_host():
    # rejected before any CUDA call: runs without a GPU
    L = _lib()
    lib = L.load()
    cap = lib.ktk_noalloc_scratch_bytes()
    assert cap == 16 << 20
    one, null = ctypes.c_void_p(16), ctypes.c_void_p(0)
    shp = _shape(4096, 1, 4, 100)                 # 4096 * 4 * 8 splits * 520 B = 68 MB > 16 MiB
    rc = lib.ktk_sparse_decode_noalloc(one, one, one, 128, one, one, 1.0, one, 8, 0, ctypes.byref(shp), null, null)
    assert rc == -5
    msg = lib.ktk_last_error().decode()
    assert "built-in" in msg and "fewer splits" in msg
    # a single split needs no scratch at all, whatever the batch: only argument checks apply
    assert lib.ktk_sparse_decode_noalloc(null, one, one, 128, one, one, 1.0, one, 1, 0, ctypes.byref(shp), null,
                                         null) == -1


def _run_pair(device, seed, lens, Hkv, G, topk, splits, variant):
    from kinetics_b200 import ops
    from oracle import oracle
    L = _lib()
    lib = L.load()
    dtype = torch.bfloat16
    q, k, v = random_case(seed, len(lens), Hkv, G, lens, dtype)
    st = paged_state(k, v, lens, dtype, seed=seed)
    d = to_dev(st, device)
    summ = oracle.summaries(st["kv_cache"], st["kv_indices"], st["kv_indptr"], st["kv_last_page_len"],
                            st["summary_stride"])
    sel, _ = oracle.select(q, summ, st["kv_indices"], st["kv_indptr"], topk)
    ref = oracle.decode(q, st["kv_cache"], sel, topk, st["kv_indptr"], st["kv_last_page_len"],
                        oracle.default_scale())
    qd, seld = q.to(device), sel.to(device)
    B, Hq = q.shape[:2]
    # 0 = the library's policy, which for bf16 is the balanced partition (KTK_SPLITS_BALANCED = -1)
    resolved = ops.decode_num_splits(B, Hkv, G, topk + 1) if splits == 0 and variant != 1 else splits
    if splits == 0 and variant != 1:
        assert resolved == ops.SPLITS_BALANCED
    ws = torch.empty(max(1, ops.decode_workspace_bytes(B, Hkv, G, resolved)), dtype=torch.uint8, device=device)
    want = ops.sparse_decode(qd, d["kv_cache"], seld, d["kv_indptr"], d["kv_last_page_len"], workspace=ws,
                             num_splits=splits, variant=variant)
    got = torch.full_like(want, float("nan"))
    shp = _shape(B, Hkv, G, st["num_pages"])
    status = ops.new_status(device)
    rc = lib.ktk_sparse_decode_noalloc(
        ctypes.c_void_p(qd.data_ptr()), ctypes.c_void_p(d["kv_cache"].data_ptr()), ctypes.c_void_p(seld.data_ptr()),
        topk, ctypes.c_void_p(d["kv_indptr"].data_ptr()), ctypes.c_void_p(d["kv_last_page_len"].data_ptr()),
        oracle.default_scale(), ctypes.c_void_p(got.data_ptr()), splits, variant, ctypes.byref(shp),
        ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.ktk_last_error().decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # same kernels, same split partition: identical bits; and within the bf16 tolerance of the oracle
    assert torch.equal(got, want)
    torch.testing.assert_close(got.float().cpu(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
def test_noalloc_decode_default_and_balanced_splits_two_calls_in_a_row(cuda_device):
    # what every bf16 caller gets without asking: num_splits = 0 resolves to the balanced partition (stream
    # kernel + combine on the built-in array); then the same partition asked for by name
    _run_pair(cuda_device, seed=73, lens=[2049, 1500, 777, 33, 4000, 16], Hkv=2, G=4, topk=48, splits=0, variant=0)
    _run_pair(cuda_device, seed=74, lens=[300, 2049, 5000], Hkv=1, G=8, topk=24, splits=-1, variant=0)


@pytest.mark.gpu
@pytest.mark.parametrize("variant", [2, 1])
def test_noalloc_decode_matches_workspace_decode_two_calls_in_a_row(cuda_device, variant):
    # first call: many splits, long lists; second call: other inputs, fewer splits, shorter lists,
    # so partial slots written by the first call lie beyond what the second one writes and reads
    _run_pair(cuda_device, seed=71, lens=[2049, 1500, 777, 33], Hkv=2, G=4, topk=48, splits=6, variant=variant)
    _run_pair(cuda_device, seed=72, lens=[300, 2049], Hkv=2, G=4, topk=24, splits=2, variant=variant)
