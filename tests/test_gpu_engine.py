"""The pooled KV manager and the engine loop on the GPU: the pool only changes WHERE pages live, so the
pooled manager must reproduce the statically paged BatchKVManager (itself checked against the oracle in
test_gpu_batch_cache.py) -- bit for bit on the sparse layers -- also while slots retire and their pages are
handed to new sequences."""
import pytest
import torch

pytestmark = pytest.mark.gpu


class Cfg:
    hidden_size = 1024
    num_attention_heads = 8
    num_key_value_heads = 2
    head_dim = 128
    num_hidden_layers = 2


def test_pooled_manager_equals_the_static_one(cuda_device):
    from kinetics_b200 import BatchKVManager, PooledKVManager
    dtype = torch.bfloat16
    kw = dict(attn_block_topk=3, attn_local=7, attn_block_size=16)
    static = BatchKVManager(Cfg, 6, 512, cuda_device, dtype, **kw)
    pooled = PooledKVManager(Cfg, 6, 512, cuda_device, dtype, num_pages=40, **kw)     # 6 x 33 pages would be 198
    g = torch.Generator().manual_seed(0)

    def rnd(*shape):
        return torch.randn(*shape, generator=g).to(dtype).to(cuda_device)

    def both(fn, bitwise=True):
        a, b = fn(static), fn(pooled)
        if bitwise:
            assert torch.equal(a, b)
        else:
            torch.testing.assert_close(a.float(), b.float(), rtol=2e-2, atol=2e-2)
        return a

    def prefill(slot, n, total):
        pooled.admit(slot, n, total)
        for layer in range(2):
            q, k, v = rnd(1, 8, n, 128), rnd(1, 2, n, 128), rnd(1, 2, n, 128)
            bi = torch.tensor([slot], device=cuda_device)
            both(lambda m: m.compute_attention(q, k, v, layer, bi))

    def decode(slots, steps):
        bi = torch.tensor(slots, device=cuda_device)
        for _ in range(steps):
            pooled.begin_step(slots)
            for layer in range(2):
                q, k, v = rnd(len(slots), 8, 1, 128), rnd(len(slots), 2, 1, 128), rnd(len(slots), 2, 1, 128)
                # layer 0 is dense (attn_layer_skip): the static manager's lists are padded rows under a
                # page_count view, the pooled one's an exact CSR, so the dense kernel cuts them at different
                # places -- same math, different rounding.  The sparse layer reads equal tables: same bits.
                both(lambda m: m.compute_attention(q, k, v, layer, bi), bitwise=(layer != 0))

    prefill(2, 150, 200)
    prefill(0, 37, 90)
    prefill(5, 3, 60)
    free0 = pooled.pool.free_pages
    decode([2, 0, 5], 20)
    # retire slot 0, hand its pages to a new sequence in slot 3, keep going with a different order of rows
    for m in (static, pooled):
        m.clear_cache(0)
    assert pooled.pool.free_pages > free0
    prefill(3, 70, 120)
    decode([5, 3, 2], 25)
    static.check_status()
    pooled.check_status()
    # the pool held far fewer pages than the static layout reserves
    assert pooled.kv_pages[0].shape[0] == 40 and static.kv_pages[0].shape[0] == 6 * static.pages_per_slot
    with pytest.raises(Exception):
        pooled.admit(1, 10, 512)                     # 33 pages: more than the pool can still promise


class TinyModel(torch.nn.Module):
    """Embedding -> 2 x (q/k/v projection, attention through the KV manager, output projection) -> logits."""

    def __init__(self, vocab, device, dtype):
        super().__init__()
        g = torch.Generator().manual_seed(5)
        mk = lambda *s: torch.nn.Parameter((torch.randn(*s, generator=g) * 0.05).to(dtype).to(device))
        self.emb = mk(vocab, Cfg.hidden_size)
        self.wq = torch.nn.ParameterList([mk(Cfg.hidden_size, 8 * 128) for _ in range(2)])
        self.wk = torch.nn.ParameterList([mk(Cfg.hidden_size, 2 * 128) for _ in range(2)])
        self.wv = torch.nn.ParameterList([mk(Cfg.hidden_size, 2 * 128) for _ in range(2)])
        self.wo = torch.nn.ParameterList([mk(8 * 128, Cfg.hidden_size) for _ in range(2)])
        self.head = mk(Cfg.hidden_size, vocab)

    @torch.inference_mode()
    def inference(self, input_ids, position_ids, batch_idx, kv):
        B, S = input_ids.shape
        x = self.emb[input_ids]                                             # [B, S, H]
        for layer in range(2):
            q = (x @ self.wq[layer]).view(B, S, 8, 128).transpose(1, 2)
            k = (x @ self.wk[layer]).view(B, S, 2, 128).transpose(1, 2)
            v = (x @ self.wv[layer]).view(B, S, 2, 128).transpose(1, 2)
            a = kv.compute_attention(q.contiguous(), k.contiguous(), v.contiguous(), layer, batch_idx)
            x = x + a.to(x.dtype) @ self.wo[layer]
        return (x @ self.head).float()


def test_engine_generates_the_same_tokens_on_a_small_pool(cuda_device):
    # greedy decoding is deterministic: a pool that forces requests to wait must not change any output
    from kinetics_b200 import BatchKVManager, Engine, PooledKVManager
    dtype, vocab = torch.float32, 97     # fp32: batch composition changes the split points, not the argmax
    model = TinyModel(vocab, cuda_device, dtype)
    g = torch.Generator().manual_seed(9)
    requests = [{"id": i, "input_ids": torch.randint(0, vocab - 1, (int(n),), generator=g).tolist()}
                for i, n in enumerate([40, 9, 130, 77, 5, 64, 23])]
    kw = dict(attn_block_topk=2, attn_local=5, attn_block_size=16)

    def run(kv):
        eng = Engine(model, kv, max_seq_len=256, device=cuda_device, temperature=0.0, eos=[vocab - 1],
                     repeat_check=False)
        out = eng.offline_exec([dict(r) for r in requests], max_new_tokens=24)
        kv.check_status()
        return {r["id"]: r["output_tokens"] for r in out}, eng

    want, _ = run(BatchKVManager(Cfg, 3, 256, cuda_device, dtype, **kw))
    small = PooledKVManager(Cfg, 3, 256, cuda_device, dtype, num_pages=22, **kw)       # 3 x 17 would be 51
    got, eng = run(small)
    assert sorted(got) == list(range(7)) and all(len(v) >= 1 for v in got.values())
    assert got == want
    assert small.pool.free_pages == 22 and not any(eng.slots_occupy_status)


def test_graphed_decode_of_a_decoder_stack_equals_the_eager_engine_step(cuda_device):
    # DecoderStack (the layer loop of litesys/models/qwen3.py on this library's ops) under Engine: prompts go
    # through the prefill kernel, then the same greedy decode steps run eagerly (Engine.decode) and with the
    # device work replayed from one CUDA graph (Engine.decode_graphed, host work in PooledKVManager.prepare_step)
    from kinetics_b200 import DecoderStack, Engine, PooledKVManager
    from kinetics_b200.config import LayerConfig
    cfg = LayerConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=512,
                      num_hidden_layers=3, vocab_size=503)
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, 500, (1, n), generator=g) for n in (150, 37, 3, 96)]
    kw = dict(attn_block_topk=3, attn_local=5, attn_block_size=16)

    def make():
        kv = PooledKVManager(cfg, 4, 256, cuda_device, dtype, num_pages=64, **kw)
        model = DecoderStack(cfg, cuda_device, dtype, max_positions=300, seed=3)
        eng = Engine(model, kv, 256, cuda_device, temperature=0.0, repeat_check=False)
        for slot, p in enumerate(prompts):
            eng.prefill(slot, p, 40)
        return eng, kv

    slots = [0, 1, 2, 3]
    eager, kv_e = make()
    graphed, kv_g = make()
    assert torch.equal(eager.slots_tokens, graphed.slots_tokens)           # same prefill, same first token
    for step in range(20):                                                 # several sequences cross page edges
        eager.decode(slots)
        out = graphed.decode_graphed(slots)
        torch.cuda.synchronize()
        n = [graphed._offsets_host[s] for s in slots]
        assert n == [eager._offsets_host[s] for s in slots]
        assert torch.equal(eager.slots_tokens, graphed.slots_tokens), step
        assert out.tolist() == [int(graphed.slots_tokens[s, n[i]]) for i, s in enumerate(slots)]
    kv_e.check_status()
    kv_g.check_status()
    assert kv_g.pool.free_pages == kv_e.pool.free_pages
