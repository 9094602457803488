"""Run under torchrun on >= 2 GPUs: the KV-head-sharded decoder layer against the unsharded layer.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 tests/multi_gpu_layer_check.py

Every rank builds the same full-size layer (TP=1) on its own GPU, runs it, then builds its shard from the
same weights and KV cache with kinetics_b200.tp and runs the N-rank layer with both exchanges (o_proj
all-reduce + residual + norm, down_proj all-reduce or reduce-scatter + residual).  The gathered N-rank
output must equal the TP=1 output within the bf16 tolerance of the path (2e-2 abs/rel), and every rank
must select, for its KV heads, the pages the full layer selects (rows whose query bits differ between the
two GEMM shapes are counted apart: their selection may legitimately differ at a near tie).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

TOL = 2e-2


def stack_logits(dev, group, steps=4):
    """A small DecoderStack (3 layers, attention through BatchKVManager): prompts through the prefill kernel,
    then `steps` batched decode steps with fixed input tokens.  Returns the logits of every call.  The page
    budget covers every page, so that a query bit that differs between the sharded and the unsharded GEMM
    cannot flip a page selection (the layer check below compares selections): what is compared here is the
    sharding of the weights, both exchanges of every layer and the head-sharded KV manager."""
    import kinetics_b200 as kb
    from kinetics_b200.config import LayerConfig
    cfg = LayerConfig(hidden_size=512, num_attention_heads=16, num_key_value_heads=8, intermediate_size=1024,
                      num_hidden_layers=3, vocab_size=1000)
    dtype = torch.bfloat16
    B = 8
    model = kb.DecoderStack(cfg, dev, dtype, process_group=group, max_positions=512, decode_batch=B, seed=5)
    kv = kb.BatchKVManager(cfg, B, 400, dev, dtype, attn_block_topk=32, attn_local=5, attn_block_size=16)
    g = torch.Generator().manual_seed(8)
    outs = []
    lens = [150, 37, 96, 3, 200, 64, 17, 81]
    for slot, n in enumerate(lens):
        ids = torch.randint(0, 1000, (1, n), generator=g).to(dev)
        pos = torch.arange(n, device=dev).unsqueeze(0)
        outs.append(model.inference(ids, pos, torch.tensor([slot], device=dev), kv)[:, -1].clone())
    bi = torch.arange(B, device=dev)
    for step in range(steps):
        ids = torch.randint(0, 1000, (B, 1), generator=g).to(dev)
        pos = torch.tensor([[n + step] for n in lens], device=dev)
        outs.append(model.inference(ids, pos, bi, kv)[:, 0].clone())
    torch.cuda.synchronize()
    kv.check_status()
    model.check_status()
    return outs


def stack_tokens(dev, group, shard_vocab, steps=3):
    """The same small stack sampling greedily through `next_tokens`, with the vocabulary projection whole on every
    rank or split by rows over the ranks (the ranks then exchange their local maxima)."""
    import kinetics_b200 as kb
    from kinetics_b200.config import LayerConfig
    cfg = LayerConfig(hidden_size=512, num_attention_heads=16, num_key_value_heads=8, intermediate_size=1024,
                      num_hidden_layers=2, vocab_size=1024)
    dtype, B = torch.bfloat16, 8
    model = kb.DecoderStack(cfg, dev, dtype, process_group=group, max_positions=512, decode_batch=B, seed=5,
                            shard_vocab=shard_vocab)
    kv = kb.BatchKVManager(cfg, B, 400, dev, dtype, attn_block_topk=32, attn_local=5, attn_block_size=16)
    g = torch.Generator().manual_seed(9)
    outs = []
    lens = [150, 37, 96, 3, 200, 64, 17, 81]
    for slot, n in enumerate(lens):
        ids = torch.randint(0, 1024, (1, n), generator=g).to(dev)
        pos = torch.arange(n, device=dev).unsqueeze(0)
        outs.append(model.next_tokens(ids, pos, torch.tensor([slot], device=dev), kv).clone())
    bi = torch.arange(B, device=dev)
    for step in range(steps):
        ids = torch.randint(0, 1024, (B, 1), generator=g).to(dev)
        pos = torch.tensor([[n + step] for n in lens], device=dev)
        outs.append(model.next_tokens(ids, pos, bi, kv).clone())
    torch.cuda.synchronize()
    kv.check_status()
    model.check_status()
    return torch.cat(outs)


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # the unsharded stack first: the KV manager reads the world size from torch.distributed, as the reference's does
    ref_logits = stack_logits(dev, None)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    import kinetics_b200 as kb
    from kinetics_b200 import tp
    from kinetics_b200.config import LayerConfig

    got_logits = stack_logits(dev, dist.group.WORLD)
    worst_stack = 0.0
    for a, b in zip(got_logits, ref_logits):
        scale = b.abs().max().item()
        err = (a - b).abs().max().item()
        assert err <= 3e-2 * max(scale, 1.0), ("decoder stack", len(got_logits), err, scale)
        worst_stack = max(worst_stack, err / max(scale, 1.0))
        same = a.clone()
        dist.broadcast(same, src=0)
        assert torch.equal(same, a), "ranks disagree on the logits"

    # greedy tokens with the vocabulary projection split over the ranks = with the whole projection on every rank
    # (the two GEMM shapes may round a logit differently: a near-tie may flip, nothing else)
    whole = stack_tokens(dev, dist.group.WORLD, False)
    split = stack_tokens(dev, dist.group.WORLD, True)
    same_tokens = (whole == split).float().mean().item()
    assert same_tokens >= 0.99, ("vocabulary-sharded greedy tokens", same_tokens)
    agreed = split.clone()
    dist.broadcast(agreed, src=0)
    assert torch.equal(agreed, split), "ranks disagree on the sampled tokens"

    cfg = LayerConfig(hidden_size=1024, num_attention_heads=32, num_key_value_heads=8, intermediate_size=2048,
                      num_hidden_layers=1)
    B, ctx, topk, dtype = 64, 2048, 16, torch.bfloat16
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim

    def build(world_size, **kw):
        layer = kb.BlockTopkDecoderLayer(cfg, world_size, B, ctx, ctx + 512, 16, topk, dev, dtype,
                                         page_table="random", seed=3, **kw)
        return layer.eval().to(dev, dtype=dtype)

    torch.manual_seed(11)                                   # the same weights, cache and input on every rank
    full = build(1)
    for name, p in full.named_parameters():
        with torch.no_grad():
            if "norm" in name:
                p.copy_((torch.rand_like(p.float()) + 0.5).to(dtype))
            else:
                p.normal_(0.0, 0.02)
    kv_before = full.kv_cache.clone()                       # the step appends a token: shards start from this
    x = torch.randn(B, 1, cfg.hidden_size, device=dev, dtype=dtype)
    full.capture = {}
    out_full = full.forward(x).clone()
    q_full = full.capture["q"]
    pages_full = full.topk_page_indices.view(B, Hkv, topk + 1).clone()
    full.check_status()

    lo, hi = tp.shard_range(Hkv, rank, world)
    g = Hq // Hkv
    lines = []
    modes = [("fused", "pipelined", "scatter"), ("fused", "pipelined", "allreduce"),
             ("fused", "lockstep", "scatter"), ("nccl", "-", "scatter"), ("nccl", "-", "allreduce")]
    for kind, schedule, down in modes:
        shard = build(world, process_group=dist.group.WORLD, fused_allreduce=(kind == "fused"),
                      down_exchange=down, kv_cache=kv_before[:, :, :, lo:hi].contiguous(),
                      **({"exchange_schedule": schedule} if kind == "fused" else {}))
        with torch.no_grad():
            w, b = tp.shard_wqkv(full.wqkv.weight, full.wqkv.bias, Hq, Hkv, D, rank, world)
            shard.wqkv.weight.copy_(w); shard.wqkv.bias.copy_(b)
            shard.wo.weight.copy_(tp.shard_wo(full.wo.weight, Hq, D, rank, world))
            u, gt, dn = tp.shard_mlp(full.up_proj.weight, full.gate_proj.weight, full.down_proj.weight, rank, world)
            shard.up_proj.weight.copy_(u); shard.gate_proj.weight.copy_(gt); shard.down_proj.weight.copy_(dn)
            for n_ in ("qnorm_weight", "knorm_weight", "input_layernorm_weight", "post_attention_layernorm_weight"):
                getattr(shard, n_).copy_(getattr(full, n_))
        shard.capture = {}
        worst = 0.0
        for step in range(3):                               # the exchanges' flags keep counting from launch to launch
            out = shard.forward(x)
            if down == "scatter":
                assert out.shape[0] == B // world
                parts = [torch.empty_like(out) for _ in range(world)]
                dist.all_gather(parts, out.contiguous())
                out = torch.cat(parts)
            torch.cuda.synchronize()
            shard.check_status()
            diff = (out.float() - out_full.float()).abs()
            bad = diff > TOL + TOL * out_full.float().abs()
            assert not bad.any(), (kind, schedule, down, step, int(bad.sum()), diff.max().item())
            worst = max(worst, diff.max().item())
            same = out.clone()
            dist.broadcast(same, src=0)
            if down == "allreduce":
                assert torch.equal(same, out), "ranks disagree on the layer output"
        # selection: rows whose query heads came out of the narrower GEMM with the same bits must pick the same pages
        q_mine = shard.capture["q"].view(B, hi - lo, g, D)
        q_ref = q_full.view(B, Hkv, g, D)[:, lo:hi]
        same_q = (q_mine == q_ref).flatten(2).all(-1)                                   # [B, local Hkv]
        pages = shard.topk_page_indices.view(B, hi - lo, topk + 1)
        same_p = (pages == pages_full[:, lo:hi]).all(-1)                                # same pages, same order
        assert bool(same_p[same_q].all()), "a row with identical query bits selected different pages"
        same_set = (pages.sort(-1).values == pages_full[:, lo:hi].sort(-1).values).all(-1)
        counts = torch.tensor([int(same_q.sum()), int(same_set.sum()), same_q.numel()], device=dev)
        dist.all_reduce(counts)
        assert counts[1].item() >= 0.95 * counts[2].item(), "selection drifted from the unsharded layer"
        lines.append(f"tp layer ok on {world} ranks: exchange {kind}/{schedule}, down_proj {down}: "
                     f"max |out - tp1| {worst:.4f}; rows with TP=1's page set {counts[1].item()}/{counts[2].item()} "
                     f"(identical query bits {counts[0].item()})")
        del shard
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("\n".join(lines), flush=True)
        print(f"tp decoder stack ok on {world} ranks: prefill + decode logits within {worst_stack:.4f} of the "
              f"unsharded stack's (relative to the largest logit), identical on every rank", flush=True)
    sys.stdout.flush()
    del full
    import gc
    gc.collect()
    from multi_gpu_allreduce_check import leave
    leave()


if __name__ == "__main__":
    main()
