"""Tensor parallelism by KV head on CPU ranks (gloo): the sharded layer equals TP=1.

Two sums cross the ranks: the o_proj partials and the down_proj partials (the MLP is column/row split);
the residual is added once after each.  The attention of each rank is the CPU oracle here -- the point is
the host-side sharding logic (which heads, which weight rows/columns, which collectives), not the kernels.
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
    import torch.nn.functional as F
    from kinetics_b200.tp import shard_mlp, shard_range, shard_wo, shard_wqkv
    from oracle.reference_layer import ReferenceLayerCPU, rmsnorm
    torch.manual_seed(0)                      # identical full-size weights and state on every rank
    Hq, Hkv, D, hid, inter, B, n = 8, 4, 128, 256, 512, 4, 12
    wq = torch.randn((Hq + 2 * Hkv) * D, hid) * 0.05
    bq = torch.randn((Hq + 2 * Hkv) * D) * 0.05
    wo = torch.randn(hid, Hq * D) * 0.05
    up, gate, down = torch.randn(inter, hid) * 0.05, torch.randn(inter, hid) * 0.05, torch.randn(hid, inter) * 0.05
    post_w = torch.rand(hid) + 0.5
    kv = torch.randn(B * (n + 1), 2, 16, Hkv, D)
    table = torch.randperm(B * (n + 1)).view(B, n + 1)
    x = torch.randn(B, 1, hid)

    def weights(wq_, bq_, wo_, up_, gate_, down_):
        return {"wqkv.weight": wq_, "wqkv.bias": bq_, "wo.weight": wo_, "up_proj.weight": up_,
                "gate_proj.weight": gate_, "down_proj.weight": down_,
                "qnorm_weight": torch.ones(D), "knorm_weight": torch.ones(D),
                "input_layernorm_weight": torch.ones(hid), "post_attention_layernorm_weight": post_w}

    def make(hq, hkv, w_, kv_):
        summ = kv_[table[:, :n], 0].mean(2).permute(0, 2, 1, 3).contiguous()
        return ReferenceLayerCPU(w_, kv_.clone(), table, summ, hq, hkv, D, 1e-6, 4)

    full_layer = make(Hq, Hkv, weights(wq, bq, wo, up, gate, down), kv)
    full = full_layer.forward(x)

    # the sharded layer, statement by statement, with the two collectives where the ranks meet
    lo, hi = shard_range(Hkv, rank, world)
    hq, hkv = Hq // world, Hkv // world
    w_ = weights(*shard_wqkv(wq, bq, Hq, Hkv, D, rank, world), shard_wo(wo, Hq, D, rank, world),
                 *shard_mlp(up, gate, down, rank, world))
    layer = make(hq, hkv, w_, kv[:, :, :, lo:hi].contiguous())
    h = rmsnorm(x, torch.ones(hid), 1e-6)
    proj = F.linear(h, w_["wqkv.weight"], w_["wqkv.bias"])
    q, k, v = proj.split((hq * D, hkv * D, hkv * D), dim=-1)
    q = rmsnorm(q.reshape(B, 1, hq, D), torch.ones(D), 1e-6).reshape(B, hq, D)
    k = rmsnorm(k.reshape(B, 1, hkv, D), torch.ones(D), 1e-6).reshape(B, hkv, D)
    layer._append(k, v.reshape(B, hkv, D))
    pages = layer._select(q)
    part = F.linear(layer._attend(q, pages).reshape(B, 1, hq * D), w_["wo.weight"])
    dist.all_reduce(part)                     # first exchange: o_proj partial sums
    resid = x + part                          # the residual is added once, after the sum
    h = rmsnorm(resid, post_w, 1e-6)
    mlp = F.linear(F.silu(F.linear(h, w_["gate_proj.weight"])) * F.linear(h, w_["up_proj.weight"]),
                   w_["down_proj.weight"])
    # second exchange: down_proj partial sums, as a reduce-scatter over the rows (rank r keeps its slice)
    per = B // world
    # (gloo has no reduce_scatter: all-reduce and slice)
    dist.all_reduce(mlp)
    mine = mlp[rank * per:(rank + 1) * per] + resid[rank * per:(rank + 1) * per]
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine.contiguous())
    got = torch.cat(gathered)
    # what a rank would return if it added the residual to its own partial and the caller summed the ranks
    wrong = world * resid + mlp
    if rank == 0:
        out.put(((full - got).abs().max().item(), (full - wrong).abs().max().item(),
                 torch.equal(full_layer.last_pages[:, lo:hi], pages)))
    dist.destroy_process_group()


def test_kv_head_sharding_with_both_exchanges_equals_the_full_layer():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err, err_wrong, same_pages = out.get(timeout=5)
    assert err < 1e-4
    assert err_wrong > 1e-2          # counting the residual once per rank is a different (wrong) result
    assert same_pages                # every rank selects, for its KV heads, the pages the full layer selects
