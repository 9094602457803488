"""The C-ABI library loads, exports what include/ktk.h declares, and validates arguments on the host."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "ktk.h").read_text()
    return sorted(set(re.findall(r"KTK_API\s+[\w\s\*]+?\b(ktk_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    from kinetics_b200 import _lib
    assert _declared() == sorted(_lib.EXPORTED)


def test_library_exports_every_declared_symbol():
    from kinetics_b200 import _lib
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in _declared():
        assert hasattr(lib, name), name
    assert _lib.load().ktk_version().decode().count(".") == 1


def _shape(**kw):
    from kinetics_b200._lib import Shape
    base = dict(batch=2, num_kv_heads=1, group_size=4, head_dim=128, page_size=16, dtype=1, num_pages=8)
    base.update(kw)
    return Shape(*[base[f] for f, _ in Shape._fields_])


def test_argument_errors_are_reported_before_any_launch():
    # every call below is rejected on the host: nothing reaches a device
    from kinetics_b200 import _lib
    lib = _lib.load()
    one = ctypes.c_void_p(16)       # a non-null dummy, never dereferenced
    null = ctypes.c_void_p(0)
    bad_head = _shape(head_dim=64)
    rc = lib.ktk_select(one, one, 4, one, one, one, 4, one, null, null, ctypes.byref(bad_head), null, null)
    assert rc == -2 and b"head_dim" in lib.ktk_last_error()
    bad_page = _shape(page_size=32)
    assert lib.ktk_append(one, one, one, one, 4, one, one, one, ctypes.byref(bad_page), null, null) == -2
    bad_group = _shape(group_size=3)
    assert lib.ktk_dense_decode(one, one, one, one, one, 4, 1.0, one, null, 0, 1, 1, ctypes.byref(bad_group),
                                null, null) == -2
    ok = _shape()
    assert lib.ktk_select(one, one, 4, one, one, one, 0, one, null, null, ctypes.byref(ok), null, null) == -1
    assert lib.ktk_select(one, one, 4, one, one, one, 5000, one, null, null, ctypes.byref(ok), null, null) == -5
    assert lib.ktk_select(null, one, 4, one, one, one, 4, one, null, null, ctypes.byref(ok), null, null) == -1
    assert lib.ktk_sparse_decode(one, one, one, 4, one, one, 1.0, one, null, 0, 3, 1, ctypes.byref(ok), null,
                                 null) == -3          # 3 splits without a workspace
    assert b"workspace" in lib.ktk_last_error()
    f32 = _shape(dtype=0)
    assert lib.ktk_sparse_decode(one, one, one, 4, one, one, 1.0, one, null, 0, 1, 2, ctypes.byref(f32), null,
                                 null) == -2          # tensor-core variant is bf16 only
    assert lib.ktk_rmsnorm(one, one, 1e-6, one, -1, 128, 1, null) == -1
    assert lib.ktk_silu_mul(one, one, one, 4, 7, null) == -1
    with pytest.raises(_lib.KtkError):
        _lib.check(-1)


def test_empty_batch_is_a_no_op():
    from kinetics_b200 import _lib
    lib = _lib.load()
    null = ctypes.c_void_p(0)
    empty = _shape(batch=0)
    assert lib.ktk_select(null, null, 0, null, null, null, 4, null, null, null, ctypes.byref(empty), null, null) == 0
    assert lib.ktk_append(null, null, null, null, 0, null, null, null, ctypes.byref(empty), null, null) == 0
    assert lib.ktk_rmsnorm(null, null, 1e-6, null, 0, 128, 1, null) == 0


def test_split_policy():
    import torch
    from kinetics_b200 import ops
    # bf16: the balanced partition, whatever the batch; its workspace does not depend on the batch
    assert ops.decode_num_splits(4096, 1, 4, 129) == ops.SPLITS_BALANCED
    assert ops.decode_num_splits(1, 1, 4, 5) == ops.SPLITS_BALANCED
    ws = ops.decode_workspace_bytes(8, 1, 4, ops.SPLITS_BALANCED)
    assert 0 < ws < (8 << 20) and ws == ops.decode_workspace_bytes(4096, 1, 4, ops.SPLITS_BALANCED)
    assert ws % (2 * 4 * 130 * 4) == 0                     # two slots per CTA, G rows of (m, l) + 128 floats
    # fp32, per-list splits.  Many sequences: one CTA each is already plenty
    assert ops.decode_num_splits(4096, 1, 4, 129, torch.float32) == 1
    # few sequences: split, but never below 8 pages per split
    s = ops.decode_num_splits(8, 1, 4, 129, torch.float32)
    assert 1 < s <= 17
    assert ops.decode_num_splits(1, 1, 4, 5, torch.float32) == 1
    assert ops.decode_workspace_bytes(8, 1, 4, 1) == 0
    assert ops.decode_workspace_bytes(8, 1, 4, 4) == 8 * 4 * 4 * 130 * 4


def test_function_level_chain_refuses_cpu_tensors():
    import torch
    from kinetics_b200 import cache_utils as cu
    k_cache = torch.zeros(2, 1, 128, 128)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        cu.copy_to_cache(k_cache, torch.zeros(1, 1, 1, 128), torch.zeros(1, dtype=torch.long),
                         torch.zeros(1, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        cu.qk(torch.zeros(1, 4, 1, 128), k_cache, torch.zeros(1, dtype=torch.long), torch.ones(1, dtype=torch.int32),
              torch.zeros(2, 4, 128), 128)
    kw = cu.preprocess_sparse_args(attn_block_topk=4, attn_local=16)
    assert kw["use_sparsity"] == 2 and kw["use_nonlocal_sparsity"] == 1 and kw["attn_layer_skip"] == [0]
    with pytest.raises(AssertionError):
        cu.preprocess_sparse_args(attn_block_topk=4)            # a non-local mask needs attn_local


def test_ops_refuse_cpu_tensors():
    import torch
    from kinetics_b200 import ops
    x = torch.zeros(4, 128)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.rmsnorm(x, torch.ones(128), 1e-6)
