"""Run under torchrun on >= 2 GPUs: the fused NVLink exchange kernels against an fp32 all-reduce + torch.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 tests/multi_gpu_allreduce_check.py

Covers both schedules (row-pipelined, lock-step), both forms (NVSwitch multicast; peer loads and stores at 2
and 4 ranks) and the three results (all-reduce + residual + RMSNorm, all-reduce + residual, reduce-scatter +
residual), several launches each so that the flag counters move on, plus the one-CTA rank barrier.
"""
import os
import sys
import threading

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def leave():
    """destroy_process_group() under a watchdog (it has been seen not to return)."""
    def give_up():
        sys.stderr.write("destroy_process_group() did not return within 20 s; leaving\n")
        sys.stderr.flush()
        os._exit(0)
    t = threading.Timer(20.0, give_up)
    t.daemon = True
    t.start()
    dist.destroy_process_group()
    t.cancel()


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from kinetics_b200 import _lib
    from kinetics_b200.comm import FusedExchange, RankBarrier

    eps = 1e-6
    forms = [("multicast", _lib.ALLREDUCE_MULTICAST)]
    if world in (2, 4):
        forms.append(("peer", _lib.ALLREDUCE_PEER))
    cases = [(schedule, result) for schedule in ("pipelined", "lockstep")
             for result in (("allreduce_norm", "allreduce", "scatter") if schedule == "pipelined" else ("allreduce_norm",))]
    worst = 0.0
    checked = 0
    # rows per rank below, at and above the number of resident CTAs (1, several and a ragged number of rows per CTA);
    # 5120 columns exercise the two-vector-per-thread kernels
    for rows, cols in ((64 * world, 4096), (40 * world * 8, 5120), (700 * world, 2048)):
        g = torch.Generator(device="cpu").manual_seed(7)         # the same residual and weight everywhere
        residual = torch.randn(rows, cols, generator=g).to(torch.bfloat16).to(dev)
        w = (torch.rand(cols, generator=g) + 0.5).to(torch.bfloat16).to(dev)
        for fname, mode in forms:
            for schedule, result in cases:
                name = f"{fname}/{schedule}/{result} {rows}x{cols}"
                ex = FusedExchange(dist.group.WORLD, rows, cols, torch.bfloat16, dev, mode=mode, result=result,
                                   schedule=schedule)
                lo, hi = ex.row_range
                for it in range(4):                                # several launches: the flags keep counting
                    torch.manual_seed(100 * it + rank)
                    part = torch.randn(rows, cols, device=dev).to(torch.bfloat16)
                    ex.x.copy_(part)
                    s, n = ex(residual, w if result == "allreduce_norm" else None, eps)
                    # reference: the fp32 sum of the partials, rounded to bf16 once (what the switch, or the
                    # peer form's fp32 accumulation, hands back), then the residual.  (A bf16 NCCL all-reduce
                    # rounds between partial sums and can be several ulps of the result away.)
                    ref = part.float()
                    dist.all_reduce(ref)
                    s_ref = (ref.to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16)
                    torch.cuda.synchronize()
                    assert int(ex.status.item()) == 0, f"{name}: a cross-rank wait ran out"
                    # the order of the fp32 additions may differ: one bf16 ulp of the partial sum (which can be much
                    # larger than the result when the residual cancels it) plus one of the result
                    tol = (ref.abs() + s_ref.float().abs()) * 2.0 ** -7 + 1e-6
                    if result == "scatter":
                        assert s.shape == (hi - lo, cols)
                        s_ref, tol = s_ref[lo:hi], tol[lo:hi]
                    bad = (s.float() - s_ref.float()).abs() > tol
                    assert not bad.any(), (name, it, int(bad.sum()), (s.float() - s_ref.float()).abs().max())
                    if result == "allreduce_norm":
                        n_ref = s_ref.float() * torch.rsqrt(s_ref.float().pow(2).mean(-1, keepdim=True) + eps) * w.float()
                        assert torch.allclose(n.float(), n_ref, rtol=2e-2, atol=2e-2), name
                    if result != "scatter":                        # every rank holds the same sum, bit for bit
                        mine = s.clone()
                        dist.broadcast(mine, src=0)
                        assert torch.equal(mine, s), f"{name}: ranks disagree on the sum"
                    worst = max(worst, (s.float() - s_ref.float()).abs().max().item())
                checked += 1
                del ex
    # the rank barrier: what a rank wrote into its peers' memory before the barrier is there after it
    from kinetics_b200.comm import SharedRows
    meet = RankBarrier(dist.group.WORLD, dev)
    rows = 8 * world
    shared = SharedRows(dist.group.WORLD, rows, 256, torch.bfloat16, dev)
    for it in range(3):
        shared.mine.fill_(float(rank + 10 * it))
        meet()
        shared.push()
        meet()
        torch.cuda.synchronize()
        per = rows // world
        want = torch.arange(world, device=dev).repeat_interleave(per).float() + 10 * it
        assert torch.equal(shared.local.float()[:, 0], want), f"all-gather by peer copies, round {it}"
        meet()                                                     # nobody overwrites a slice that is still being checked
    assert int(meet.status.item()) == 0
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"fused exchange ok on {world} ranks, {checked} kernel variants, max |sum - ref| {worst:.4f}", flush=True)
    sys.stdout.flush()
    del meet, shared
    leave()


if __name__ == "__main__":
    main()
