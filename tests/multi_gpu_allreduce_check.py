"""Run under torchrun on >= 2 GPUs: the fused multicast all-reduce + add + RMSNorm against NCCL + torch.

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

    rows, cols, eps = 64 * world, 4096, 1e-6
    fused = FusedAllReduceNorm(dist.group.WORLD, rows, cols, torch.bfloat16, dev)
    g = torch.Generator(device="cpu").manual_seed(7)             # the same residual and weight everywhere
    residual = torch.randn(rows, cols, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.rand(cols, generator=g) + 0.5).to(torch.bfloat16).to(dev)
    worst = 0.0
    for it in range(5):                                            # several launches: the flags keep counting
        torch.manual_seed(100 * it + rank)
        part = torch.randn(rows, cols, device=dev).to(torch.bfloat16)
        fused.x.copy_(part)
        s, n = fused(residual, w, eps)
        ref = part.clone()
        dist.all_reduce(ref)
        s_ref = (ref.float() + residual.float()).to(torch.bfloat16)
        n_ref = s_ref.float() * torch.rsqrt(s_ref.float().pow(2).mean(-1, keepdim=True) + eps) * w.float()
        torch.cuda.synchronize()
        assert int(fused.status.item()) == 0, "a cross-rank wait ran out"
        # the switch sums in fp32 and rounds once, NCCL may round between partial sums: one bf16 ulp apart at most
        assert torch.allclose(s.float(), s_ref.float(), rtol=2e-2, atol=2e-2), (s.float() - s_ref.float()).abs().max()
        assert torch.allclose(n.float(), n_ref, rtol=2e-2, atol=2e-2)
        worst = max(worst, (s.float() - s_ref.float()).abs().max().item())
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"fused all-reduce ok on {world} ranks, max |sum - ref| {worst:.4f}", flush=True)
    if os.environ.get("KTK_TIME_ALLREDUCE"):
        # the layer's shape: 4096 x 4096 bf16 = 32 MiB per rank
        from kinetics_b200 import ops
        big = FusedAllReduceNorm(dist.group.WORLD, 4096, 4096, torch.bfloat16, dev)
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

        t_fused = timed(lambda: big(res, wb, eps))

        def nccl_path():
            dist.all_reduce(part)
            ops.add_rmsnorm(part, res, wb, eps)

        t_nccl = timed(nccl_path)
        if rank == 0:
            print(f"32 MiB: fused kernel {t_fused * 1e3:.1f} us, NCCL all-reduce + add_rmsnorm {t_nccl * 1e3:.1f} us", flush=True)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
