"""Decoder layers on the GPU against the reference's forward restated on CPU tensors."""
import pytest
import torch

from oracle import oracle
from oracle.reference_layer import ReferenceLayerCPU

pytestmark = pytest.mark.gpu


class Cfg:
    hidden_size = 512
    num_attention_heads = 8
    num_key_value_heads = 2
    head_dim = 128
    intermediate_size = 1024
    rms_norm_eps = 1e-6
    hidden_act = "silu"
    rope_theta = 1e6
    max_position_embeddings = 4096
    eos_token_id = 0
    num_hidden_layers = 1


def _weights(layer):
    sd = {k: v.detach().float().cpu() for k, v in layer.state_dict().items()}
    return sd


def _build(cls, device, dtype, **kw):
    import kinetics_b200 as kb
    torch.manual_seed(0)
    layer = getattr(kb, cls)(config=Cfg, world_size=1, batch_size=6, prefix_len=40 * 16, max_len=40 * 16 + 64,
                             page_size=16, device=device, dtype=dtype, **kw)
    layer.apply(kb.init_weights)
    layer.eval()
    layer.to(device, dtype=dtype)
    return layer


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("table", ["interleaved", "random"])
def test_blocktopk_layer_matches_reference_forward(cuda_device, dtype, table):
    layer = _build("BlockTopkDecoderLayer", cuda_device, dtype, topk_page=8, page_table=table, seed=3)
    cache_before = layer.kv_cache.float().cpu()
    summ_before = layer.compressed_key_cache.float().cpu()
    x = torch.randn(6, 1, Cfg.hidden_size, device=cuda_device, dtype=dtype)
    layer.capture = {}
    y = layer(x)
    layer.check_status()
    ref = ReferenceLayerCPU(_weights(layer), cache_before.clone(), layer.page_table.cpu(), summ_before.clone(),
                            8, 2, 128, Cfg.rms_norm_eps, 8)
    if dtype == torch.bfloat16:
        # the fp32 restatement sees a slightly different q than the bf16 layer and may rank two close
        # pages the other way round: let it attend the pages the layer picked (checked below)
        ref.forced_pages = layer.topk_page_indices.view(6, 2, 9).long().cpu()
    y_ref = ref.forward(x.float().cpu())
    # the pages the kernel picked are the oracle's pick for the q the GPU actually produced
    q = layer.capture["q"].cpu()
    cache_after = layer.kv_cache.cpu()
    summ_after = layer.compressed_key_cache.cpu()
    phys, _ = oracle.select(q, summ_after, layer.paged_kv_indices.cpu(), layer.full_kv_indptr.cpu(), 8)
    assert torch.equal(layer.topk_page_indices.view(6, 2, 9).cpu(), phys)
    # appended token landed in slot 0 of each sequence's last page, summaries follow
    last_pages = layer.page_table[:, -1].long().cpu()
    assert torch.equal(cache_after[last_pages, 0, 0], layer.capture["k"].cpu())
    assert torch.equal(cache_after[last_pages, 1, 0], layer.capture["v"].cpu())
    assert torch.equal(summ_after[:, :, 40], layer.capture["k"].cpu())
    tol = 2e-3 if dtype == torch.float32 else 6e-2
    if dtype == torch.float32:
        # same q up to GEMM rounding: same page sets unless a near tie, so compare outputs directly
        assert torch.equal(torch.sort(ref.last_pages, -1).values, torch.sort(phys.long(), -1).values)
    torch.testing.assert_close(y.float().cpu(), y_ref, rtol=tol, atol=tol)


def test_dense_and_sparse_layers_share_a_process_and_a_cache(cuda_device):
    dtype = torch.bfloat16
    sparse = _build("BlockTopkDecoderLayer", cuda_device, dtype, topk_page=64)       # budget >= pages: dense
    dense = _build("DecoderLayer", cuda_device, dtype, kv_cache=sparse.kv_cache)
    dense.load_state_dict(sparse.state_dict())
    # same page list, same split count => the two paths run the very same arithmetic
    sparse.decode_plan.num_splits = 1
    dense.decode_plan.num_splits = 1
    x = torch.randn(6, 1, Cfg.hidden_size, device=cuda_device, dtype=dtype)
    a = sparse(x)
    b = dense(x)
    torch.testing.assert_close(a, b, rtol=0, atol=0)


def test_graph_replay_equals_eager(cuda_device):
    dtype = torch.bfloat16
    layer = _build("BlockTopkDecoderLayer", cuda_device, dtype, topk_page=8)
    x = torch.randn(6, 1, Cfg.hidden_size, device=cuda_device, dtype=dtype)
    eager = layer(x).clone()
    static_in, static_out, graph = layer.make_graphed(x)
    graph.replay()
    torch.cuda.synchronize()
    torch.testing.assert_close(static_out, eager, rtol=0, atol=0)
    layer.check_status()


def test_ragged_contexts_select_like_the_oracle(cuda_device):
    # The Qwen3-32B ragged configuration in small: ragged per-sequence contexts, fragmented page pool
    import kinetics_b200 as kb
    dtype = torch.bfloat16
    torch.manual_seed(0)
    lens = [40 * 16, 17, 16, 0, 333, 100]
    layer = kb.BlockTopkDecoderLayer(config=Cfg, world_size=1, batch_size=6, prefix_len=40 * 16, max_len=40 * 16 + 64,
                                     page_size=16, topk_page=8, device=cuda_device, dtype=dtype, page_table="random",
                                     seed=5, context_lens=lens)
    layer.apply(kb.init_weights)
    layer.eval()
    layer.to(cuda_device, dtype=dtype)
    assert (layer.full_kv_indptr[1:] - layer.full_kv_indptr[:-1]).tolist() == [n // 16 + 1 for n in lens]
    x = torch.randn(6, 1, Cfg.hidden_size, device=cuda_device, dtype=dtype)
    layer.capture = {}
    y = layer(x)
    layer.check_status()
    assert torch.isfinite(y).all()
    q = layer.capture["q"].cpu()
    phys, _ = oracle.select(q, layer.compressed_key_cache.cpu(), layer.paged_kv_indices.cpu(),
                            layer.full_kv_indptr.cpu(), 8)
    assert torch.equal(layer.topk_page_indices.view(6, 2, 9).cpu(), phys)
    ref = oracle.decode(q, layer.kv_cache.cpu(), phys, 8, layer.full_kv_indptr.cpu(), layer.last_kv_lens.cpu(),
                        oracle.default_scale())
    got = kb.ops.sparse_decode(layer.capture["q"], layer.kv_cache, layer.topk_page_indices.view(6, 2, 9),
                               layer.full_kv_indptr, layer.last_kv_lens, num_splits=1)
    torch.testing.assert_close(got.float().cpu(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_qkv_norm_with_rotary_embedding(cuda_device, dtype):
    # split + q-norm + k-norm + rotary embedding in one launch, against the reference's statements in fp32
    # (LiteSys/litesys/models/qwen3.py:96-102, models/model_utils.py:17-50)
    import kinetics_b200 as kb
    g = torch.Generator().manual_seed(17)
    B, Hq, Hkv, D, eps, max_pos = 37, 8, 2, 128, 1e-6, 500
    proj = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(dtype).to(cuda_device)
    wq = (torch.rand(D, generator=g) + 0.5).to(dtype).to(cuda_device)
    wk = (torch.rand(D, generator=g) + 0.5).to(dtype).to(cuda_device)
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.outer(torch.arange(max_pos).float(), inv_freq)
    emb = torch.cat([ang, ang], dim=-1)
    cos, sin = emb.cos().to(dtype).to(cuda_device), emb.sin().to(dtype).to(cuda_device)
    pos = torch.randint(0, max_pos, (B,), generator=g).to(cuda_device)
    q, k, v = kb.ops.qkv_norm(proj, wq, wk, eps, Hq, Hkv, cos=cos, sin=sin, position_ids=pos)

    def norm(x, w):
        x = x.float()
        return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(dtype).float()

    def rope(x):
        c, s = cos[pos].float()[:, None, :], sin[pos].float()[:, None, :]
        rot = torch.cat([-x[..., D // 2:], x[..., :D // 2]], dim=-1)
        return x * c + rot * s

    p3 = proj.view(B, Hq + 2 * Hkv, D)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(q.float(), rope(norm(p3[:, :Hq], wq)), rtol=tol, atol=tol)
    torch.testing.assert_close(k.float(), rope(norm(p3[:, Hq:Hq + Hkv], wk)), rtol=tol, atol=tol)
    assert torch.equal(v, p3[:, Hq + Hkv:])
    # without tables the kernel is the plain split + norms
    q0, k0, v0 = kb.ops.qkv_norm(proj, wq, wk, eps, Hq, Hkv)
    torch.testing.assert_close(q0.float(), norm(p3[:, :Hq], wq), rtol=tol, atol=tol)
    assert torch.equal(v0, v)
