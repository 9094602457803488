"""The boundary under the reference's own launcher: benchmark/blocktopk.py:41-43 wraps the layer's forward in
torch.compile(..., fullgraph=True), which only works if every step of the forward is a registered torch op
with a fake (meta) implementation (benchmark/blocktopk_decoder.py:23-85, :171-184)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _layer(cls, device, **kw):
    from kinetics_b200.config import LayerConfig
    cfg = LayerConfig(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, intermediate_size=1024,
                      num_hidden_layers=1)
    torch.manual_seed(5)
    layer = cls(config=cfg, world_size=1, batch_size=8, prefix_len=1024, max_len=1536, page_size=16, device=device,
                dtype=torch.bfloat16, page_table="random", seed=2, **kw)
    for m in layer.modules():
        if isinstance(m, torch.nn.Linear):
            torch.nn.init.normal_(m.weight, 0.0, 0.05)
            torch.nn.init.normal_(m.bias, 0.0, 0.05) if m.bias is not None else None
    return layer.eval().to(device, dtype=torch.bfloat16), cfg


@pytest.mark.parametrize("sparse", [True, False])
def test_compiled_forward_equals_eager(cuda_device, sparse):
    import kinetics_b200 as kb
    layer, cfg = _layer(kb.BlockTopkDecoderLayer if sparse else kb.DecoderLayer, cuda_device,
                        **({"topk_page": 8} if sparse else {}))
    x = torch.randn(8, 1, cfg.hidden_size, device=cuda_device, dtype=torch.bfloat16)
    eager = layer.forward(x).clone()
    pages = layer.topk_page_indices.clone() if sparse else None
    compiled = torch.compile(layer.forward, fullgraph=True)       # raises on any graph break
    if sparse:
        layer.prepare_wrapper(1024)                                # as the reference does after compiling
    else:
        layer.prepare_wrapper()
    out = compiled(x)
    out2 = compiled(x)
    layer.check_status()
    # the custom ops are the same kernels; only the glue around the GEMMs may be fused differently
    torch.testing.assert_close(out.float(), eager.float(), rtol=2e-2, atol=2e-2)
    assert torch.equal(out, out2)
    if sparse:
        assert torch.equal(layer.topk_page_indices, pages)


def test_opcheck_of_the_reference_named_ops(cuda_device):
    import kinetics_b200 as kb
    from kinetics_b200 import ops
    layer, cfg = _layer(kb.BlockTopkDecoderLayer, cuda_device, topk_page=8)
    B, Hq, Hkv = 8, layer.num_heads, layer.num_kv_heads
    dt = torch.bfloat16
    q = torch.randn(B, Hq, 128, device=cuda_device, dtype=dt)
    k = torch.randn(B, Hkv, 128, device=cuda_device, dtype=dt)
    v = torch.randn(B, Hkv, 128, device=cuda_device, dtype=dt)
    w = torch.rand(128, device=cuda_device, dtype=dt) + 0.5
    layer.forward(torch.randn(B, 1, cfg.hidden_size, device=cuda_device, dtype=dt))      # binds plan and summaries
    checks = ("test_schema", "test_faketensor")
    torch.library.opcheck(torch.ops.mylib.update_kv.default,
                          (k, v, layer.qkv_indptr, layer.kv_cache, layer.paged_kv_indices, layer.full_kv_indptr,
                           layer.last_kv_lens), test_utils=checks)
    torch.library.opcheck(torch.ops.mylib.decode.default, (q, layer.kv_cache), test_utils=checks)
    torch.library.opcheck(torch.ops.mylib.qk_norm.default, (q, 1e-6, w), test_utils=checks)
    x = torch.randn(B, cfg.hidden_size, device=cuda_device, dtype=dt)
    wl = torch.rand(cfg.hidden_size, device=cuda_device, dtype=dt) + 0.5
    torch.library.opcheck(torch.ops.mylib.layer_norm.default, (x, 1e-6, wl), test_utils=checks)
    # the added ops of the fused glue and the selection
    torch.library.opcheck(torch.ops.ktk.rms_norm.default, (x, wl, 1e-6), test_utils=checks)
    torch.library.opcheck(torch.ops.ktk.add_rms_norm.default, (x, x.clone(), wl, 1e-6), test_utils=checks)
    proj = torch.randn(B, (Hq + 2 * Hkv) * 128, device=cuda_device, dtype=dt)
    torch.library.opcheck(torch.ops.ktk.qkv_norm.default, (proj, w, w, 1e-6, Hq, Hkv), test_utils=checks)
    torch.library.opcheck(torch.ops.ktk.silu_mul.default, (x, x.clone()), test_utils=checks)
    out = torch.empty(B, Hkv, 9, dtype=torch.int32, device=cuda_device)
    torch.library.opcheck(torch.ops.ktk.select_pages_into.default,
                          (q, layer.compressed_key_cache, layer.paged_kv_indices, layer.full_kv_indptr,
                           layer.last_kv_lens, 8, layer.total_pages, out, ops.new_status(cuda_device)),
                          test_utils=checks)
    layer.check_status()


def test_bindings_go_with_the_layer(cuda_device):
    import gc
    import kinetics_b200 as kb
    from kinetics_b200 import ops
    layer, _ = _layer(kb.BlockTopkDecoderLayer, cuda_device, topk_page=8)
    address = layer.kv_cache.data_ptr()
    assert address in ops._PLANS and address in ops._SUMMARIES
    del layer
    gc.collect()
    assert address not in ops._PLANS and address not in ops._SUMMARIES
