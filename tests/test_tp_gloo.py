"""Tensor parallelism by KV head on CPU ranks (gloo): the sum of the ranks' o_proj partials equals TP=1.

The attention of each rank is the CPU oracle here -- the point is the host-side sharding logic
(which heads, which weight rows/columns, which collective), not the kernels.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from kinetics_b200.tp import shard_range, shard_wo, shard_wqkv
    from oracle.reference_layer import ReferenceLayerCPU
    torch.manual_seed(0)                      # identical full-size weights and state on every rank
    Hq, Hkv, D, hid, B, n = 8, 4, 128, 256, 3, 12
    wq = torch.randn((Hq + 2 * Hkv) * D, hid) * 0.05
    bq = torch.randn((Hq + 2 * Hkv) * D) * 0.05
    wo = torch.randn(hid, Hq * D) * 0.05
    kv = torch.randn(B * (n + 1), 2, 16, Hkv, D)
    table = torch.randperm(B * (n + 1)).view(B, n + 1)
    x = torch.randn(B, 1, hid)

    def attn_out(hq, hkv, wq_, bq_, wo_, kv_):
        summ = kv_[table[:, :n], 0].mean(2).permute(0, 2, 1, 3).contiguous()
        layer = ReferenceLayerCPU({"wqkv.weight": wq_, "wqkv.bias": bq_, "wo.weight": wo_,
                                   "qnorm_weight": torch.ones(D), "knorm_weight": torch.ones(D),
                                   "input_layernorm_weight": torch.ones(hid)}, kv_.clone(), table, summ,
                                  hq, hkv, D, 1e-6, 4)
        # the attention half of the forward, up to the o_proj partial
        from oracle.reference_layer import rmsnorm
        import torch.nn.functional as F
        h = rmsnorm(x, torch.ones(hid), 1e-6)
        proj = F.linear(h, wq_, bq_)
        q, k, v = proj.split((hq * D, hkv * D, hkv * D), dim=-1)
        q = rmsnorm(q.reshape(B, 1, hq, D), torch.ones(D), 1e-6).reshape(B, hq, D)
        k = rmsnorm(k.reshape(B, 1, hkv, D), torch.ones(D), 1e-6).reshape(B, hkv, D)
        layer._append(k, v.reshape(B, hkv, D))
        pages = layer._select(q)
        return F.linear(layer._attend(q, pages).reshape(B, 1, hq * D), wo_)

    full = attn_out(Hq, Hkv, wq, bq, wo, kv)
    lo, hi = shard_range(Hkv, rank, world)
    part = attn_out(Hq // world, Hkv // world, *shard_wqkv(wq, bq, Hq, Hkv, D, rank, world),
                    shard_wo(wo, Hq, D, rank, world), kv[:, :, :, lo:hi].contiguous())
    dist.all_reduce(part)                     # the one collective of the path (o_proj partial sums)
    if rank == 0:
        out.put((full - part).abs().max().item())
    dist.destroy_process_group()


def test_kv_head_sharding_sums_to_full_layer():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(timeout=5) < 1e-4
