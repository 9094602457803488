"""Run under torchrun on >= 2 GPUs: the fused all-reduce + add + RMSNorm (both forms) against an fp32 all-reduce + torch.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 tests/multi_gpu_allreduce_check.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from kinetics_b200.comm import FusedAllReduceNorm

    from kinetics_b200 import _lib
    rows, cols, eps = 64 * world, 4096, 1e-6
    modes = [("multicast", _lib.ALLREDUCE_MULTICAST)]
    if world in (2, 4):
        modes.append(("peer", _lib.ALLREDUCE_PEER))
    g = torch.Generator(device="cpu").manual_seed(7)             # the same residual and weight everywhere
    residual = torch.randn(rows, cols, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.rand(cols, generator=g) + 0.5).to(torch.bfloat16).to(dev)
    worst = 0.0
    for name, mode in modes:
        fused = FusedAllReduceNorm(dist.group.WORLD, rows, cols, torch.bfloat16, dev, mode=mode)
        for it in range(5):                                        # several launches: the flags keep counting
            torch.manual_seed(100 * it + rank)
            part = torch.randn(rows, cols, device=dev).to(torch.bfloat16)
            fused.x.copy_(part)
            s, n = fused(residual, w, eps)
            # reference: the fp32 sum of the partials, rounded to bf16 once (what the switch, or the
            # peer form's fp32 accumulation, hands back), then the residual.  (A bf16 NCCL all-reduce
            # rounds between partial sums and can be several ulps of the result away.)
            ref = part.float()
            dist.all_reduce(ref)
            s_ref = (ref.to(torch.bfloat16).float() + residual.float()).to(torch.bfloat16)
            n_ref = s_ref.float() * torch.rsqrt(s_ref.float().pow(2).mean(-1, keepdim=True) + eps) * w.float()
            torch.cuda.synchronize()
            assert int(fused.status.item()) == 0, f"{name}: a cross-rank wait ran out"
            # the order of the fp32 additions may differ: one bf16 ulp of the partial sum (which can be much
            # larger than the result when the residual cancels it) plus one of the result
            tol = (ref.abs() + s_ref.float().abs()) * 2.0 ** -7 + 1e-6
            bad = (s.float() - s_ref.float()).abs() > tol
            assert not bad.any(), (name, int(bad.sum()), (s.float() - s_ref.float()).abs().max())
            assert torch.allclose(n.float(), n_ref, rtol=2e-2, atol=2e-2), name
            # every rank holds the same sum, bit for bit
            mine = s.clone()
            dist.broadcast(mine, src=0)
            assert torch.equal(mine, s), f"{name}: ranks disagree on the sum"
            worst = max(worst, (s.float() - s_ref.float()).abs().max().item())
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"fused all-reduce ok on {world} ranks, max |sum - ref| {worst:.4f}", flush=True)
    if os.environ.get("KTK_TIME_ALLREDUCE"):
        # the layer's shape: 4096 x 4096 bf16 = 32 MiB per rank
        from kinetics_b200 import ops
        res = torch.randn(4096, 4096, device=dev).to(torch.bfloat16)
        wb = torch.ones(4096, device=dev, dtype=torch.bfloat16)
        part = torch.randn(4096, 4096, device=dev).to(torch.bfloat16)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def timed(fn, n=50):
            for _ in range(5):
                fn()
            dist.barrier(); torch.cuda.synchronize()
            e0.record()
            for _ in range(n):
                fn()
            e1.record(); torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n

        t_fused = {}
        for name, mode in modes:
            big = FusedAllReduceNorm(dist.group.WORLD, 4096, 4096, torch.bfloat16, dev, mode=mode)
            t_fused[name] = timed(lambda: big(res, wb, eps))

        def nccl_path():
            dist.all_reduce(part)
            ops.add_rmsnorm(part, res, wb, eps)

        t_nccl = timed(nccl_path)
        if rank == 0:
            fused_txt = ", ".join(f"fused kernel ({k}) {v * 1e3:.1f} us" for k, v in t_fused.items())
            print(f"32 MiB: {fused_txt}, NCCL all-reduce + add_rmsnorm {t_nccl * 1e3:.1f} us", flush=True)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
