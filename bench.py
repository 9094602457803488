#!/usr/bin/env python
"""Benchmark of the block top-k decode layer (one JSON line on stdout).

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W    # the reference's path on host cores

Workload (default ``cfg3-shard``): one Qwen3-8B-shaped decoder layer at the paper's throughput shape
-- batch 4096, 32768-token context, page size 16, block top-k budget of 128 pages, bf16 -- sharded
8-way by KV head the way the reference benchmark does it (``--world_size 8``: one KV head, four
query heads and 1/8 of the MLP per GPU, benchmark/blocktopk_decoder.py:101-106).  Every rank of an
N-GPU run holds one such shard (weak scaling) and sums the o_proj partial results with the ranks' fused
all-reduce + residual + RMSNorm kernel over NVLink (``--allreduce nccl`` for NCCL instead).
A step is one forward of the layer: RMSNorm, QKV projection, q/k-norm, paged append (+ page
summary), page scoring + top-k selection, attention over the selected pages, o_proj (+ all-reduce),
MLP.  The reported value is decode tokens/s in full-layer equivalents, ``batch * N / 8 / t_step``:
with 8 ranks it is the throughput of the whole layer, with one rank it is the number the
reference prints times its layer count (benchmark/blocktopk.py:82).

Synthetic data: KV cache and hidden states N(0,1), weights N(0, 0.02), seeded.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # the paper's throughput shape (Qwen3-8B, batch 4096, 32768-token context) as one 8-way KV-head shard per GPU (68.2 GB of KV per GPU)
    "cfg3-shard": dict(model="Qwen3-8B", tp=8, batch=4096, ctx=32768, topk=128),
    # Qwen3-8B, batch 256, 8192-token context, top-k 64: at TP=8 (one shard) and TP=1
    "cfg2-shard": dict(model="Qwen3-8B", tp=8, batch=256, ctx=8192, topk=64),
    "cfg2-tp1": dict(model="Qwen3-8B", tp=1, batch=256, ctx=8192, topk=64),
    # the Qwen3-32B shape with uniform context (ragged contexts are covered by the parity tests)
    "cfg4-shard": dict(model="Qwen3-32B", tp=8, batch=1024, ctx=8192, topk=64),
    # Qwen3-32B: ragged contexts uniform in [1024, 16384], fragmented (randomly permuted) page pool, GQA 8
    "cfg4-ragged": dict(model="Qwen3-32B", tp=8, batch=1024, ctx=16384, topk=64, ragged=(1024, 16384)),
    # one Qwen3-1.7B layer (GQA 2, all 8 KV heads on one GPU), 512 sequences with contexts uniform in
    # [512, 32768]; a tenth of them sit on a page boundary, so the step opens a new page for those
    "cfg5-tp1": dict(model="Qwen3-1.7B", tp=1, batch=512, ctx=32768, topk=32, ragged=(512, 32768), boundary=0.1),
    "tiny": dict(model="Qwen3-8B", tp=8, batch=64, ctx=2048, topk=16),
    # the whole Qwen3-1.7B model (28 layers, final norm, vocabulary projection, greedy
    # sampling) stepping 512 sequences with contexts uniform in [512, 32768], a tenth of them on a page boundary
    # at the first timed step, block top-k budget 32; tensor parallel over the GPUs of the run (--gpus 1/2/4/8),
    # driven by Engine + PagePool (the page table is exported on the host every step)
    "cfg5": dict(model="Qwen3-1.7B", tp=0, batch=512, ctx=32768, topk=32, ragged=(512, 32768), boundary=0.1,
                 full_model=True),
    # the CPU-runnable reference case: fp32, one KV head with four query heads, 4 sequences of 2048 tokens, top-k 16
    "cfg1": dict(model="cfg1", tp=1, batch=4, ctx=2048, topk=16, dtype="float32"),
}
PAGE = 16
HEAD_DIM = 128
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_stream_kernel launch over its algorithmic bytes,
# from a profiler capture of the same kernel and shape at batch 296 (one CTA per resident slot, every page
# read once: the traffic grows with the batch in proportion)
DECODE_TRAFFIC_RATIO = 1.016
DECODE_TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of decode_stream_kernel at batch 296 of "
                         "this shape = 1.016 x algorithmic bytes, applied to this run's bytes")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3-shard", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch size")
    ap.add_argument("--variant", type=int, default=0, help="decode kernel: 0 auto, 1 fp32-FMA, 2 tensor-core")
    ap.add_argument("--splits", type=int, default=0, help="decode split count (0 = library policy)")
    ap.add_argument("--no-dense", action="store_true", help="skip the dense paged decode comparison")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--page-table", default="interleaved", choices=["interleaved", "random"])
    ap.add_argument("--seed", type=int, default=1236)
    ap.add_argument("--cpu-sample", type=int, default=32, help="sequences in the CPU sample")
    ap.add_argument("--allreduce", default="auto", choices=["auto", "fused", "nccl"],
                    help="N > 1: sum the o_proj partials with the fused multicast kernel (all-reduce + residual add "
                         "+ RMSNorm in one launch: peer loads at 2 and 4 ranks, NVSwitch multicast above), or with NCCL "
                         "followed by the add + norm kernel.  auto: fused")
    ap.add_argument("--down-exchange", default="scatter", choices=["scatter", "allreduce"],
                    help="N > 1: what the down_proj exchange leaves on a rank: its row slice of the layer output "
                         "(reduce-scatter + residual) or all rows (all-reduce + residual, the reference's form)")
    ap.add_argument("--exchange-schedule", default=None, choices=["pipelined", "lockstep"],
                    help="schedule of the fused o_proj exchange kernel (default: by size, lock-step above 8 MiB)")
    ap.add_argument("--reps", type=int, default=5, help="repetitions of the --steps loop; the median is reported")
    ap.add_argument("--no-flashinfer", action="store_true",
                    help="skip the library comparison.  By default a one-GPU run also times, on the same cache and "
                         "lists, the library kernels the reference uses on a GPU: flashinfer's paged batch decode "
                         "(sparse list and dense table) and the reference's torch selection statements; reported "
                         "under \"library_bar\", never part of the headline")
    ap.add_argument("--flashinfer", action="store_true", help="(default now; kept for old command lines)")
    ap.add_argument("--flashinfer-cuda-cores", action="store_true",
                    help="library comparison: also flashinfer's CUDA-core decode (one more kernel to build)")
    ap.add_argument("--library-timeout", type=float, default=420.0,
                    help="seconds the library comparison may take (flashinfer builds its kernels on first use)")
    ap.add_argument("--layers", type=int, default=0, help="full-model workloads: run this many layers (0: all)")
    ap.add_argument("--one-rank-of", type=int, default=0,
                    help="full-model workloads on one GPU: run the compute of ONE rank of this many (heads and MLP "
                         "width divided, no exchange) -- what a step costs without the NVLink exchanges")
    ap.add_argument("--prefill-tokens", type=int, default=4096, help="--micro prefill: new tokens per prompt")
    ap.add_argument("--prefill-history", type=int, default=0,
                    help="--micro prefill: tokens every prompt already holds in its pages (a later chunk of a long prompt)")
    ap.add_argument("--micro", default="", choices=["", "select", "exchange", "prefill"],
                    help="time one kernel alone on the workload's shapes (select: only the page summaries are "
                         "allocated, so the full batch fits in a few GB; exchange: the NVLink exchange kernels "
                         "on [batch, hidden] under torchrun, every form, beside NCCL)")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------
# clocks (read-only NVML sampling during the timed regions)
# ------------------------------------------------------------------------------------------

class ClockSampler:
    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.sm, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    _NAMES = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
              0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
              0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.sm.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self._NAMES.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None
        return False

    def summary(self):
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.sm)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------------------------------------
# CPU baseline: the reference's layer forward on host cores, bounded sample of the workload
# ------------------------------------------------------------------------------------------

def cpu_reference_run(wl, sample_batch: int, steps: int, warmup: int, seed: int, budget_s: float = 20.0):
    """Times oracle/reference_layer.py (torch on CPU, all host threads) on `sample_batch` sequences of the
    workload's shape.  Returns (tokens_per_s in full-layer equivalents, ms_per_step, threads, steps_run)."""
    # by path: importing the package would map libktk.so, which has no part in this arm
    import importlib.util
    spec = importlib.util.spec_from_file_location("_ktk_config", os.path.join(ROOT, "kinetics_b200", "config.py"))
    cfgmod = importlib.util.module_from_spec(spec)
    sys.modules["_ktk_config"] = cfgmod
    spec.loader.exec_module(cfgmod)
    get_config = cfgmod.get_config
    from oracle.reference_layer import ReferenceLayerCPU

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    cfg = get_config(wl["model"])
    tp = wl["tp"]
    hq, hkv, inter, hid = cfg.num_attention_heads // tp, cfg.num_key_value_heads // tp, cfg.intermediate_size // tp, cfg.hidden_size
    n = wl["ctx"] // PAGE
    B = sample_batch
    g = torch.Generator().manual_seed(seed)
    dt = torch.float32

    def w(*shape):
        return torch.empty(*shape, dtype=dt).normal_(0, 0.02, generator=g)

    weights = {
        "wqkv.weight": w((hq + 2 * hkv) * HEAD_DIM, hid), "wqkv.bias": w((hq + 2 * hkv) * HEAD_DIM),
        "wo.weight": w(hid, hq * HEAD_DIM), "up_proj.weight": w(inter, hid), "gate_proj.weight": w(inter, hid),
        "down_proj.weight": w(hid, inter), "qnorm_weight": torch.ones(HEAD_DIM), "knorm_weight": torch.ones(HEAD_DIM),
        "input_layernorm_weight": torch.ones(hid), "post_attention_layernorm_weight": torch.ones(hid),
    }
    pages = B * (n + 1)
    kv = torch.empty(pages, 2, PAGE, hkv, HEAD_DIM, dtype=dt).normal_(generator=g)
    table = (torch.arange(n + 1)[None, :] * B + torch.arange(B)[:, None])
    summ = kv[table[:, :n], 0].mean(2).permute(0, 2, 1, 3).contiguous()          # [B, Hkv, n, D]
    layer = ReferenceLayerCPU(weights, kv, table, summ, hq, hkv, HEAD_DIM, cfg.rms_norm_eps, wl["topk"])
    x = torch.empty(B, 1, hid, dtype=dt).normal_(generator=g)
    for _ in range(max(1, warmup)):
        layer.forward(x)
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        layer.forward(x)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt_s = (time.perf_counter() - t0) / done
    return B / tp / dt_s, dt_s * 1e3, threads, done


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = dict(WORKLOADS[args.workload])
    if args.batch:
        wl["batch"] = args.batch
    args.cpu_sample = min(args.cpu_sample, wl["batch"])
    value, ms, threads, done = cpu_reference_run(wl, args.cpu_sample, args.steps, args.warmup, args.seed,
                                                 budget_s=120.0)
    sample = (f"{args.cpu_sample} of {wl['batch']} sequences of the workload per step, fp32, "
              f"torch on {threads} host threads")
    line = {
        "impl": "reference", "metric": "block-top-k decode tokens/s (Qwen3-8B layer, B=4096, 32K ctx)",
        "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": done, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": dict(workload_config(args, wl, args.gpus), sample_batch=args.cpu_sample),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def use_fused_allreduce(args, world):
    if world < 2 or args.allreduce == "nccl":
        return False
    return True


def workload_config(args, wl, n_gpus):
    return {
        "workload": (f"{args.workload}: {wl['model']} decoder layer, "
                     + (f"{wl['tp']}-way KV-head shard per GPU" if wl["tp"] > 1 else "all KV heads on one GPU")
                     + f" (tp={wl['tp']}), batch {wl['batch']}, context "
                     + (f"uniform in {list(wl['ragged'])}" if "ragged" in wl else str(wl["ctx"]))
                     + f", page {PAGE}, top-k {wl['topk']} pages, one decode step"),
        "batch": wl["batch"], "context": wl["ctx"], "page_size": PAGE, "topk_pages": wl["topk"],
        "tp_shards_total": wl["tp"], "shards_resident": n_gpus, "page_table": args.page_table,
        "l2": "per-step traffic (summaries + selected pages) exceeds the 126 MB L2; no flush needed",
        "parallelism": f"tp{wl['tp']} by KV head, {n_gpus} shard(s) resident, o_proj all-reduce: "
                       + (("fused kernel (all-reduce + add + RMSNorm), "
                           + ("peer loads and stores" if n_gpus in (2, 4) else "NVSwitch multicast"))
                          if use_fused_allreduce(args, n_gpus) else "NCCL")
                       if n_gpus > 1 else f"tp{wl['tp']} by KV head, 1 shard resident",
    }


# ------------------------------------------------------------------------------------------
# the reference's GPU statements and library, for comparison (not the product, not the headline)
# ------------------------------------------------------------------------------------------

def library_bar_run(layer, hidden, B, hkv, hq, topk, device, with_dense=True, iters=10, cuda_cores=False):
    """Times, with CUDA events, what the reference executes on a GPU for the same step:
    its selection statements in torch (benchmark/blocktopk_decoder.py:216-221, one KV head) and
    flashinfer's BatchDecodeWithPagedKVCacheWrapper (:153-160,176-178,255-265) over the selected list and,
    for the dense layer (dense_decoder.py:149-156,168-170), over the whole page table."""
    import flashinfer
    layer.capture = {}
    layer.forward(hidden)
    q = layer.capture["q"].contiguous()                        # [B, Hq, D]
    layer.capture = None
    n = layer.num_pages_per_req
    G = hq // hkv
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    out = {"flashinfer": flashinfer.__version__}
    summ = layer.compressed_key_cache[:, 0, :n].contiguous()   # [B, n, D], KV head 0
    qg = q.view(B, hkv, G, -1)[:, 0]                           # [B, G, D]
    table = layer.page_table.long()                            # [B, n+1]

    def torch_select():
        csim = torch.einsum("bgd,bnd->bgn", qg, summ).mean(dim=1)
        idx = csim.topk(k=topk, dim=-1).indices
        phys = torch.gather(table[:, :n], 1, idx)
        return torch.cat([phys, table[:, n:]], dim=-1).to(torch.int32)

    out["torch_select_ms"] = timed(torch_select)
    ws = torch.empty(128 * 1024 * 1024, dtype=torch.uint8, device=device)
    sel = layer.topk_page_indices.view(B, hkv, topk + 1)[:, 0].contiguous().view(-1)
    sel_indptr = torch.arange(B + 1, dtype=torch.int32, device=device) * (topk + 1)
    for name, tc in ((("cuda_cores", False),) if cuda_cores else ()) + (("tensor_cores", True),):
        try:
            w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD", use_tensor_cores=tc)
            w.plan(sel_indptr, sel, layer.last_kv_lens, hq, hkv, HEAD_DIM, PAGE, pos_encoding_mode="NONE",
                   q_data_type=q.dtype, kv_data_type=layer.kv_cache.dtype)
            out[f"flashinfer_sparse_decode_ms_{name}"] = timed(lambda: w.run(q, layer.kv_cache))
            if with_dense:
                w.plan(layer.full_kv_indptr, layer.paged_kv_indices, layer.last_kv_lens, hq, hkv, HEAD_DIM, PAGE,
                       pos_encoding_mode="NONE", q_data_type=q.dtype, kv_data_type=layer.kv_cache.dtype)
                out[f"flashinfer_dense_decode_ms_{name}"] = timed(lambda: w.run(q, layer.kv_cache))
        except Exception as e:                                  # the library could not build or run its kernel
            out[f"flashinfer_{name}_error"] = str(e)[:200]
    return out


# ------------------------------------------------------------------------------------------
# this repository's path
# ------------------------------------------------------------------------------------------

def mean_ms(pairs):
    return sum(a.elapsed_time(b) for a, b in pairs) / max(len(pairs), 1)


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def sampled_attention_check(layer, hidden, rows: int = 64, seed: int = 0):
    """One eager forward with the layer's intermediate tensors kept; for `rows` sampled sequences the
    attention output of every local KV head is recomputed in fp32 torch over the pages the step selected
    (last page masked to its fill level), and the selection is recomputed as the reference states it
    (benchmark/blocktopk_decoder.py:216-217: einsum, mean over the group, k largest) in fp32."""
    layer.capture = {}
    layer.forward(hidden)
    torch.cuda.synchronize()
    q, o = layer.capture["q"].float(), layer.capture["o"].float()          # [B, Hq, D]
    layer.capture = None
    B, hkv, k1 = layer.batch_size, layer.num_kv_heads, layer.topk_page + 1
    G = layer.num_key_value_groups
    sel = layer.topk_page_indices.view(B, hkv, k1)
    gsel = torch.Generator().manual_seed(seed)
    picks = torch.randperm(B, generator=gsel)[:rows].tolist()
    indptr = layer.full_kv_indptr.tolist()
    worst, pages_checked, sets_equal, set_rows = 0.0, 0, 0, 0
    for b in picks:
        n_pages = indptr[b + 1] - indptr[b]
        n_scored = n_pages - 1
        cnt = min(layer.topk_page, n_scored) + 1
        last = int(layer.last_kv_lens[b])
        table = layer.paged_kv_indices[indptr[b]:indptr[b + 1]].long()
        for h in range(hkv):
            pages = sel[b, h, :cnt].long()
            kv = layer.kv_cache[pages][:, :, :, h].float()                  # [cnt, 2, P, D]
            ntok = (cnt - 1) * PAGE + last
            kk = kv[:, 0].reshape(cnt * PAGE, HEAD_DIM)[:ntok]
            vv = kv[:, 1].reshape(cnt * PAGE, HEAD_DIM)[:ntok]
            qg = q[b, h * G:(h + 1) * G]
            p_ = torch.softmax(qg @ kk.t() / HEAD_DIM ** 0.5, dim=-1)
            ref = p_ @ vv
            worst = max(worst, (ref - o[b, h * G:(h + 1) * G]).abs().max().item())
            pages_checked += cnt
            if n_scored > layer.topk_page:
                summ = layer.compressed_key_cache[b, h, :n_scored].float()
                csim = torch.einsum("gd,nd->gn", qg, summ).mean(0)
                want = set(table[csim.topk(layer.topk_page).indices].tolist())
                sets_equal += int(want == set(pages[:-1].tolist()))
                set_rows += 1
    return {"rows": len(picks), "kv_heads": hkv, "pages_checked": pages_checked, "max_abs_err": worst,
            "tolerance": 2e-2, "selected_sets_equal_torch_fp32": f"{sets_equal}/{set_rows}",
            "how": "fp32 torch attention over the pages the step selected; selection vs einsum+mean+topk in fp32"}


def run_ours(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this path has no CPU fallback (use --impl reference)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    pg = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        pg = dist.group.WORLD

    import kinetics_b200 as kb
    from kinetics_b200 import ops

    wl = dict(WORKLOADS[args.workload])
    if args.batch:
        wl["batch"] = args.batch
    cfg = kb.get_config(wl["model"])
    tp, B, ctx, topk = wl["tp"], wl["batch"], wl["ctx"], wl["topk"]
    dtype = getattr(torch, wl.get("dtype", "bfloat16"))
    torch.manual_seed(args.seed * 1000 + rank)
    fused = use_fused_allreduce(args, world)
    scatter = world > 1 and args.down_exchange == "scatter"

    ctx_lens = None
    if "ragged" in wl:
        lo, hi = wl["ragged"]
        gl = torch.Generator().manual_seed(args.seed)            # the same lengths on every rank
        ctx_lens = torch.randint(lo, hi + 1, (B,), generator=gl)
        on_boundary = int(round(wl.get("boundary", 0.0) * B))
        if on_boundary:
            pick = torch.randperm(B, generator=gl)[:on_boundary]
            ctx_lens[pick] = ctx_lens[pick] // PAGE * PAGE
        args.page_table = "random"

    def make(cls, **kw):
        if world > 1:
            kw.update(down_exchange=args.down_exchange, exchange_schedule=args.exchange_schedule)
        layer = cls(config=cfg, world_size=tp, batch_size=B, prefix_len=ctx, max_len=ctx + 512, page_size=PAGE,
                    device=device, dtype=dtype, page_table=args.page_table, process_group=pg,
                    seed=args.seed + rank, variant=args.variant, context_lens=ctx_lens,
                    fused_allreduce=fused, **kw)
        for m in layer.modules():
            if isinstance(m, torch.nn.Linear):
                torch.nn.init.normal_(m.weight, 0.0, 0.02)
                if m.bias is not None:
                    torch.nn.init.normal_(m.bias, 0.0, 0.02)
        layer.eval()
        layer.to(device, dtype=dtype)
        return layer

    sparse = make(kb.BlockTopkDecoderLayer, topk_page=topk)
    sparse.decode_plan.num_splits = args.splits
    hidden = torch.randn(B, 1, cfg.hidden_size, device=device, dtype=dtype)
    if world > 1:
        dist.broadcast(hidden, src=0)                            # tensor parallelism replicates the hidden states
    static_in, static_out, graph = sparse.make_graphed(hidden)
    sparse.check_status()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local)

    # ---- timed region: `reps` passes of K graph replays, inputs resident in HBM; the median pass is the value ----
    for _ in range(args.warmup):
        graph.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    passes = []
    with sampler:
        for _ in range(max(1, args.reps)):
            e0.record()
            for _ in range(args.steps):
                graph.replay()
            e1.record()
            barrier()
            passes.append(max_over_ranks(e0.elapsed_time(e1) / args.steps))
    ms_step = median(passes)
    value = B * world / tp / (ms_step * 1e-3)

    # ---- per-kernel durations, CUDA events around each of our kernels in an eager pass ----
    sparse.timers = {}
    ksteps = max(5, min(args.steps, 50))
    launches0 = ops.launch_count()
    with sampler:
        for _ in range(ksteps):
            sparse.forward(static_in)
        torch.cuda.synchronize()
    launches_per_step = (ops.launch_count() - launches0) // ksteps
    timers, sparse.timers = sparse.timers, None
    t_select = mean_ms(timers["select"][2:])
    t_decode = mean_ms(timers["decode"][2:])
    t_append = mean_ms(timers["append"][2:])
    hkv = cfg.num_key_value_heads // tp
    esz = 2 if dtype == torch.bfloat16 else 4
    scored = (ctx_lens // PAGE) if ctx_lens is not None else torch.full((B,), ctx // PAGE)
    bytes_select = int(scored.sum()) * hkv * HEAD_DIM * esz
    bytes_decode = int((torch.clamp(scored, max=topk) + 1).sum()) * hkv * PAGE * HEAD_DIM * 2 * esz
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    ach_decode = bytes_decode / (t_decode * 1e-3) / 1e9
    ach_select = bytes_select / (t_select * 1e-3) / 1e9
    ach_attn = (bytes_decode + bytes_select) / ((t_decode + t_select) * 1e-3) / 1e9
    # DRAM traffic of one launch of the decode kernel: not measurable inside this run (it needs the
    # profiler), so the ratio of a profiler capture of the same kernel is applied to this run's bytes.
    traffic = int(bytes_decode * DECODE_TRAFFIC_RATIO) if dtype == torch.bfloat16 else None
    roofline = {"bound": "hbm", "kernel": "sparse decode (decode_stream_kernel + stream_combine_kernel)"
                if dtype == torch.bfloat16 else "sparse decode (decode_simt_kernel, fp32)",
                "achieved": ach_decode, "peak": peak_gbs, "unit": "GB/s", "frac": ach_decode / peak_gbs,
                "traffic": traffic, "traffic_source": DECODE_TRAFFIC_SOURCE,
                "peak_kind": peak_kind, "ms": t_decode, "algorithmic_bytes": bytes_decode}
    kernels = {
        "select": {"ms": t_select, "algorithmic_bytes": bytes_select, "achieved_gbs": ach_select,
                   "frac": ach_select / peak_gbs},
        "decode": {"ms": t_decode, "algorithmic_bytes": bytes_decode, "achieved_gbs": ach_decode,
                   "frac": ach_decode / peak_gbs},
        "append": {"ms": t_append},
        "attention_total": {"ms": t_select + t_decode, "achieved_gbs": ach_attn, "frac": ach_attn / peak_gbs,
                            "frac_of_8TBs_nominal": ach_attn / 8000.0},
    }
    if world > 1:
        # the two exchanges as the eager pass saw them (a rank's wait for the slowest rank included)
        hid_bytes = B * cfg.hidden_size * esz
        for name in ("exchange_o_proj", "exchange_down_proj"):
            if name in timers:
                t = max_over_ranks(mean_ms(timers[name][2:]))
                kernels[name] = {"ms": t, "payload_bytes": hid_bytes}
        kernels["exchange_exposed_ms_per_step"] = sum(kernels[n]["ms"] for n in ("exchange_o_proj", "exchange_down_proj")
                                                      if n in kernels)

    # ---- the attention kernels back to back inside a CUDA graph, as they run in the step ----
    # Events around eager launches include the host's launch gaps, which for 20-100 us kernels are as long as
    # the kernels.  Here select -> decode (+ combine) repeat `inner` times in one graph on the step's own query;
    # one iteration moves summaries + selected pages (more than the L2 holds for every workload but the tiny
    # ones), so each select streams its summaries from HBM again, as in the step.
    sparse.capture = {}
    sparse.forward(static_in)
    q_step = sparse.capture["q"].contiguous()
    sparse.capture = None
    inner = 20
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        sparse._attention(q_step)
    torch.cuda.current_stream().wait_stream(side)
    g_attn = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_attn):
        for _ in range(inner):
            sparse._attention(q_step)
    for _ in range(3):
        g_attn.replay()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(5):
        g_attn.replay()
    e1.record()
    torch.cuda.synchronize()
    t_attn_graph = e0.elapsed_time(e1) / (5 * inner)
    ach_graph = (bytes_decode + bytes_select) / (t_attn_graph * 1e-3) / 1e9
    kernels["attention_total_in_graph"] = {
        "ms": t_attn_graph, "achieved_gbs": ach_graph, "frac": ach_graph / peak_gbs,
        "frac_of_8TBs_nominal": ach_graph / 8000.0,
        "how": f"select + decode (+ combine) x {inner} in one CUDA graph, 5 replays, per iteration"}
    del g_attn

    # ---- the attention output of the step against fp32 torch over the pages it selected (sampled rows) ----
    parity = sampled_attention_check(sparse, static_in) if rank == 0 or world > 1 else None

    # ---- end to end: host buffers in, host buffers out, every step ----
    # Three streams: the next step's input is copied in and the previous step's output is copied
    # out while the current step computes; two captured graphs alternate so that each has its own
    # input buffer.
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, sparse, hidden, (static_in, static_out, graph), world, rank, pg, device, B, cfg, dtype,
                      tp, sampler, barrier, max_over_ranks, scatter)
    sparse.check_status()

    # ---- the repository's dense paged decode at the same shape, sharing the KV cache ----
    dense_info = None
    if not args.no_dense:
        dense = make(kb.DecoderLayer, kv_cache=sparse.kv_cache)
        dense.timers = {}
        dsteps = 4
        for _ in range(2):
            dense.forward(static_in)
        barrier()
        e0.record()
        for _ in range(dsteps):
            dense.forward(static_in)
        e1.record()
        barrier()
        ms_dense = max_over_ranks(e0.elapsed_time(e1) / dsteps)
        t_dd = mean_ms(dense.timers["decode"][2:])
        dense.timers = None
        bytes_dense = int((scored + 1).sum()) * hkv * PAGE * HEAD_DIM * 2 * esz
        dense_info = {"tokens_per_s": B * world / tp / (ms_dense * 1e-3), "ms_per_step": ms_dense,
                      "decode_ms": t_dd, "decode_gbs": bytes_dense / (t_dd * 1e-3) / 1e9,
                      "sparse_over_dense": ms_dense / ms_step}
        dense.check_status()
        del dense

    # ---- the library kernels the reference itself runs on a GPU, on the same cache (comparison only) ----
    library_bar = None
    if not args.no_flashinfer and world == 1 and ctx_lens is None and dtype == torch.bfloat16:
        library_bar = bounded_library_bar(args, sparse, static_in, B, hkv, cfg.num_attention_heads // tp, topk, device,
                                          with_dense=not args.no_dense)
        if library_bar and "flashinfer_sparse_decode_ms_tensor_cores" in library_bar:
            lib_sel = library_bar["torch_select_ms"]
            lib_dec = library_bar["flashinfer_sparse_decode_ms_tensor_cores"]
            vs = {"select": lib_sel / t_select, "sparse_decode": lib_dec / t_decode,
                  "select_plus_sparse_decode": (lib_sel + lib_dec) / (t_select + t_decode)}
            if dense_info and "flashinfer_dense_decode_ms_tensor_cores" in library_bar:
                vs["dense_decode"] = library_bar["flashinfer_dense_decode_ms_tensor_cores"] / dense_info["decode_ms"]
            library_bar["vs_library"] = dict(vs, meaning="library time / this repository's time (> 1: faster here)")

    # ---- CPU baseline (rank 0, single-GPU run only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and ctx_lens is None:
        sys.path.insert(0, ROOT)
        sample_b = min(args.cpu_sample, B)
        v, ms, threads, done = cpu_reference_run(wl, sample_b, 1000, 1, args.seed, budget_s=15.0)
        cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "ms_per_step": ms,
               "sample": f"{sample_b} of {B} sequences of the workload per step, {done} steps, fp32, "
                         f"torch on {threads} host threads (oracle/reference_layer.py)"}

    if rank == 0:
        line = {
            "metric": "block-top-k decode tokens/s (Qwen3-8B layer, B=4096, 32K ctx)", "value": value,
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "ms_per_step_passes": {"reps": len(passes), "min": min(passes), "median": ms_step, "max": max(passes)},
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dtype == torch.bfloat16 else "f32", "data": "synthetic",
            "config": workload_config(args, wl, world), "roofline": roofline, "kernels": kernels,
            "parity_check": parity, "cpu_baseline": cpu, "e2e": e2e, "dense": dense_info,
            "library_bar": library_bar,
            "gpu_launches": launches_per_step * args.steps * max(1, args.reps),
            "gpu_launches_per_step": launches_per_step,
            # what benchmark/blocktopk.py:60,82 prints for one shard: B / t / (world_size * num_hidden_layers)
            "reference_normalisation": {"tokens_per_s": B / (ms_step * 1e-3) / (tp * cfg.num_hidden_layers),
                                        "world_size": tp, "num_hidden_layers": cfg.num_hidden_layers},
            "clocks": sampler.summary(),
        }
        emit(line)
    if world > 1:
        leave_group(dist, [graph, sparse])


def leave_group(dist, holders):
    """Tear the process group down after the graphs and exchange buffers that use it are gone.  A watchdog
    ends the process if the teardown does not return (it has been seen to wait forever with captured
    graphs alive); every rank has finished its work once it passes the barrier."""
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    holders.clear()
    import gc
    gc.collect()
    torch.cuda.synchronize()

    def give_up():
        sys.stderr.write("bench.py: destroy_process_group() did not return within 20 s; leaving\n")
        sys.stderr.flush()
        os._exit(0)

    t = threading.Timer(20.0, give_up)
    t.daemon = True
    t.start()
    dist.destroy_process_group()
    t.cancel()


def run_e2e(args, sparse, hidden, first_set, world, rank, pg, device, B, cfg, dtype, tp, sampler, barrier,
            max_over_ranks, scatter):
    H = cfg.hidden_size
    s_in, s_out, s_comp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world == 1:
        sets = [first_set, sparse.make_graphed(hidden)]
        host_in = [torch.randn(B, 1, H, dtype=dtype).pin_memory() for _ in range(2)]
        host_out = [torch.empty(B, 1, H, dtype=dtype).pin_memory() for _ in range(2)]

        def run_steps(n):
            ev_in = [None, None]; ev_comp = [None, None]; ev_out = [None, None]
            for i in range(n):
                j = i & 1
                buf_in, buf_out, g = sets[j]
                with torch.cuda.stream(s_in):
                    if ev_comp[j] is not None:
                        s_in.wait_event(ev_comp[j])          # the graph that read this buffer has finished
                    buf_in.copy_(host_in[j], non_blocking=True)
                    ev_in[j] = torch.cuda.Event(); ev_in[j].record(s_in)
                s_comp.wait_event(ev_in[j])
                if ev_out[j] is not None:
                    s_comp.wait_event(ev_out[j])             # its previous output has left the device
                g.replay()
                ev_comp[j] = torch.cuda.Event(); ev_comp[j].record(s_comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[j])
                    host_out[j].copy_(buf_out, non_blocking=True)
                    ev_out[j] = torch.cuda.Event(); ev_out[j].record(s_out)
            s_comp.wait_stream(s_out)
            s_comp.wait_stream(s_in)

        nbytes_in = nbytes_out = host_in[0].numel() * host_in[0].element_size()
        how = ("pinned host input -> device, layer step, output -> pinned host, every step; copies of "
               "neighbouring steps overlap the compute on separate streams")
    else:
        # Tensor parallelism replicates the hidden states, so the host data is split by rows instead: rank r
        # copies rows [r*B/N, (r+1)*B/N) of the step's input from its pinned host memory, the ranks hand their
        # slices to one another with copy-engine peer copies (an all-gather that needs no SM), and each rank
        # copies back the row slice of the layer output it owns after the down_proj reduce-scatter.  Two
        # one-CTA barrier kernels per step order the peer copies against the other ranks' graphs.
        from kinetics_b200.comm import RankBarrier, SharedRows
        per = B // world
        shared = [SharedRows(pg, B, H, dtype, device) for _ in range(2)]
        meet = RankBarrier(pg, device)
        sets = []
        for j in range(2):
            shared[j].local.copy_(hidden.view(B, H))
            g_in, g_out, g = sparse.make_graphed(hidden, static_in=shared[j].local.view(B, 1, H))
            sets.append((g_in, g_out, g))
        r0 = rank * per
        host_in = [torch.randn(per, H, dtype=dtype).pin_memory() for _ in range(2)]
        host_out = [torch.empty(per, H, dtype=dtype).pin_memory() for _ in range(2)]
        stage_out = [torch.empty(per, H, dtype=dtype, device=device) for _ in range(2)]

        def run_steps(n):
            ev_in = [None, None]; ev_comp = [None, None]; ev_out = [None, None]
            for i in range(n):
                j = i & 1
                _, buf_out, g = sets[j]
                with torch.cuda.stream(s_in):
                    if ev_comp[j] is not None:
                        s_in.wait_event(ev_comp[j])          # this rank's graph that read the buffer has finished
                    shared[j].mine.copy_(host_in[j], non_blocking=True)
                    meet()                                   # ... and so has every other rank's
                    shared[j].push()
                    meet()                                   # every rank's slice has landed here
                    ev_in[j] = torch.cuda.Event(); ev_in[j].record(s_in)
                s_comp.wait_event(ev_in[j])
                if ev_out[j] is not None:
                    s_comp.wait_event(ev_out[j])             # the staging buffer has left the device
                g.replay()
                out_rows = buf_out.view(-1, H) if scatter else buf_out.view(B, H)[r0:r0 + per]
                stage_out[j].copy_(out_rows, non_blocking=True)      # the exchange's output buffer is reused next step
                ev_comp[j] = torch.cuda.Event(); ev_comp[j].record(s_comp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp[j])
                    host_out[j].copy_(stage_out[j], non_blocking=True)
                    ev_out[j] = torch.cuda.Event(); ev_out[j].record(s_out)
            s_comp.wait_stream(s_out)
            s_comp.wait_stream(s_in)

        nbytes_in = nbytes_out = world * host_in[0].numel() * host_in[0].element_size()
        how = ("every rank copies its row slice of the step's input from pinned host memory, the slices are "
               "all-gathered with copy-engine peer copies between two barrier kernels, layer step, every rank "
               "copies its row slice of the output back; neighbouring steps overlap on separate streams")

    run_steps(4)
    barrier()
    with sampler:
        e0.record()
        run_steps(args.steps)
        e1.record()
        barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    if world > 1:
        ops_mod = __import__("kinetics_b200").ops
        ops_mod.raise_on_status(meet.status)
    return {"value": B * world / tp / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
            "h2d_bytes_per_step": nbytes_in, "d2h_bytes_per_step": nbytes_out, "how": how}


def bounded_library_bar(args, layer, hidden, B, hkv, hq, topk, device, with_dense):
    """library_bar_run in a worker thread with a time limit: flashinfer compiles its kernels with nvcc on
    first use, which can take minutes on a fresh machine."""
    box = {}

    def work():
        try:
            torch.cuda.set_device(device)
            box["out"] = library_bar_run(layer, hidden, B, hkv, hq, topk, device, with_dense=with_dense,
                                         cuda_cores=args.flashinfer_cuda_cores)
        except Exception as e:                                  # the library is missing or could not build
            box["out"] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}

    t = threading.Thread(target=work, daemon=True)
    t.start()
    t.join(args.library_timeout)
    if t.is_alive():
        return {"skipped": f"the library comparison did not finish within {args.library_timeout:.0f} s "
                           "(flashinfer builds its kernels on first use)"}
    return box.get("out")


def run_micro_select(args):
    """The scoring + selection kernel alone at the workload's shape (no KV cache is needed for it)."""
    from kinetics_b200 import ops
    import kinetics_b200 as kb
    wl = dict(WORKLOADS[args.workload])
    if args.batch:
        wl["batch"] = args.batch
    cfg = kb.get_config(wl["model"])
    B, topk = wl["batch"], wl["topk"]
    tp = args.one_rank_of or wl.get("tp") or 1
    hkv, hq = cfg.num_key_value_heads // tp, cfg.num_attention_heads // tp
    dev = torch.device("cuda", 0)
    torch.manual_seed(args.seed)
    if "ragged" in wl:                                       # contexts uniform in [lo, hi], like the workload's
        lo, hi = wl["ragged"]
        scored = (torch.randint(lo, hi + 1, (B,), generator=torch.Generator().manual_seed(args.seed)) // PAGE).to(dev)
    else:
        scored = torch.full((B,), wl["ctx"] // PAGE, device=dev)
    n = int(scored.max())
    dtype = torch.bfloat16
    summ = torch.randn(B, hkv, n + 32, HEAD_DIM, device=dev, dtype=dtype)
    q = torch.randn(B, hq, HEAD_DIM, device=dev, dtype=dtype)
    indptr = torch.zeros(B + 1, dtype=torch.int32, device=dev)
    indptr[1:] = torch.cumsum(scored + 1, 0)                 # the scored pages + the page being filled
    total_pages = int(indptr[-1])
    table = torch.arange(total_pages, dtype=torch.int32, device=dev)
    last = torch.ones(B, dtype=torch.int32, device=dev)
    out = torch.empty(B, hkv, topk + 1, dtype=torch.int32, device=dev)
    status = ops.new_status(dev)
    # each launch timed by its own pair of events, with a write larger than L2 before it
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(view):
        run = lambda: ops.select_pages(q, summ, table, indptr, last, topk, total_pages, out=out, status=status,
                                       view=view)
        for _ in range(args.warmup):
            run()
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                 for _ in range(args.steps)]
        for e0, e1 in pairs:
            flush.zero_()
            e0.record()
            run()
            e1.record()
        torch.cuda.synchronize()
        ops.raise_on_status(status)
        return median([e0.elapsed_time(e1) for e0, e1 in pairs])

    ms = timed(None)
    # the same with the sequences handed to the CTAs from the longest to the shortest
    order = torch.argsort(scored, descending=True, stable=True).to(torch.int32)
    ms_ordered = timed(ops.PageView(0, 1, None, None, order))
    nbytes = int(scored.sum()) * hkv * HEAD_DIM * 2
    emit({"micro": "select", "batch": B, "kv_heads": hkv, "pages_scored_max": n, "topk": topk, "ms": ms,
          "ms_with_seq_order": ms_ordered,
          "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / (ms * 1e-3) / 1e9})


def run_micro_prefill(args):
    """Causal prefill attention alone: `--batch` prompts (default 4) of `--prefill-tokens` tokens, the workload's heads
    per rank, bf16, no history.  Times the tcgen05 kernel (the default) and the mma.sync kernel it replaced."""
    from kinetics_b200 import ops, _lib
    import kinetics_b200 as kb
    wl = dict(WORKLOADS[args.workload])
    cfg = kb.get_config(wl["model"])
    tp = args.one_rank_of or wl.get("tp") or 1
    hkv, hq = cfg.num_key_value_heads // tp, cfg.num_attention_heads // tp
    B, n, hist = args.batch or 4, args.prefill_tokens, args.prefill_history
    dev = torch.device("cuda", 0)
    torch.manual_seed(args.seed)
    pages_per = (hist + n + PAGE - 1) // PAGE
    cache = torch.randn(B * pages_per, 2, PAGE, hkv, HEAD_DIM, device=dev).to(torch.bfloat16)
    q = torch.randn(B * n, hq, HEAD_DIM, device=dev).to(torch.bfloat16)
    indptr = torch.arange(B + 1, dtype=torch.int32, device=dev) * pages_per
    table = torch.arange(B * pages_per, dtype=torch.int32, device=dev)
    last = torch.full((B,), hist + n - (pages_per - 1) * PAGE, dtype=torch.int32, device=dev)
    q_indptr = torch.arange(B + 1, dtype=torch.int32, device=dev) * n
    status = ops.new_status(dev)
    flop = B * hq * (n * hist + n * (n + 1) / 2) * HEAD_DIM * 4      # QK^T and PV over history + causal half
    out, outs = {"micro": "prefill", "prompts": B, "tokens": n, "history": hist, "kv_heads": hkv, "q_heads": hq, "causal_flop": flop,
                 "kernels": {}}, {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, variant in (("prefill_umma_kernel (tcgen05)", _lib.VARIANT_UMMA), ("prefill_mma_kernel (mma.sync)", _lib.VARIANT_MMA)):
        run = lambda: ops.prefill_attention(q, q_indptr, n, cache, table, indptr, last, variant=variant, status=status)
        for _ in range(max(3, args.warmup)):
            outs[variant] = run()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        out["kernels"][name] = {"ms": ms, "tflops": flop / (ms * 1e-3) / 1e12}
    ops.raise_on_status(status)
    out["max_abs_difference_between_the_two"] = float(
        (outs[_lib.VARIANT_UMMA].float() - outs[_lib.VARIANT_MMA].float()).abs().max())
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops", 1590.0))
    out["peak_tflops"] = peak
    out["frac"] = out["kernels"]["prefill_umma_kernel (tcgen05)"]["tflops"] / peak
    emit(out)


def run_full_model(args):
    """A full-model decode step (Qwen3-1.7B, 512 sequences in continuous batching).  One process per GPU; the model is tensor parallel
    over the ranks of the run.  A step = Engine.decode_graphed: host page-table work (PagePool growth, CSR export,
    asynchronous copies into static device buffers) + one CUDA-graph replay of embedding, 28 layers (block top-k
    attention through PooledKVManager, LiteSys semantics: sink 4, layer 0 dense), final norm, vocabulary
    projection, argmax and token bookkeeping."""
    import torch.distributed as dist
    import numpy as np

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    pg = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        pg = dist.group.WORLD
    import kinetics_b200 as kb
    from kinetics_b200 import ops

    wl = dict(WORKLOADS[args.workload])
    if args.batch:
        wl["batch"] = args.batch
    cfg = kb.get_config(wl["model"])
    shard_of = args.one_rank_of if world == 1 else 0
    if shard_of > 1:
        import dataclasses
        cfg = dataclasses.replace(cfg, num_attention_heads=cfg.num_attention_heads // shard_of,
                                  num_key_value_heads=cfg.num_key_value_heads // shard_of,
                                  intermediate_size=cfg.intermediate_size // shard_of)
    B, topk = wl["batch"], wl["topk"]
    lo, hi = wl["ragged"]
    dtype = torch.bfloat16
    layers = args.layers or cfg.num_hidden_layers
    gl = torch.Generator().manual_seed(args.seed)
    lens = torch.randint(lo, hi + 1, (B,), generator=gl)
    on_boundary = int(round(wl.get("boundary", 0.0) * B))
    pick = torch.randperm(B, generator=gl)[:on_boundary]
    # a sequence opens a page when the token it appends is the first behind a page edge (4 sink tokens, then 16s)
    ahead = 2 + max(args.warmup, 3)                          # decode steps that run before the first timed one
    lens[pick] = torch.clamp((lens[pick] - 4) // PAGE * PAGE + 4 - ahead, min=lo)
    steps_total = args.warmup + args.steps * max(1, args.reps) * 2 + 16
    max_seq = int(lens.max()) + steps_total + PAGE
    pool_pages = int(((lens + steps_total - 4 + PAGE - 1) // PAGE + 2).sum()) + 64
    hkv = cfg.num_key_value_heads // world
    kv_bytes_layer = pool_pages * 2 * PAGE * hkv * HEAD_DIM * 2
    # every layer needs its own pages; they fit only when the model is spread over enough GPUs
    alias = kv_bytes_layer * layers > 140e9
    torch.manual_seed(args.seed)

    class Cfg:                                               # what the KV manager reads from a model config
        hidden_size, num_attention_heads, num_key_value_heads = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads
        head_dim, num_hidden_layers = cfg.head_dim, layers

    kv = kb.PooledKVManager(Cfg, B, max_seq, device, dtype, num_pages=pool_pages, alias_layers=alias,
                            attn_block_topk=topk, attn_local=0, attn_block_size=PAGE)
    for pages in ({id(p): p for p in kv.kv_pages}.values()):
        pages.normal_()                                      # KV pre-filled from N(0, 1)
    kv.assume_filled({s: int(lens[s]) for s in range(B)}, headroom=steps_total)
    # greedy sampling: the argmax is taken over the bf16 logits (identical to the argmax of an fp32 copy)
    model = kb.DecoderStack(cfg, device, dtype, process_group=pg, max_positions=max_seq + 8, decode_batch=B,
                            seed=args.seed, num_layers=layers, logits_dtype=None, shard_vocab=world > 1)
    eng = kb.Engine(model, kv, max_seq, device, temperature=0.0, repeat_check=False)
    slots = list(range(B))
    for s in slots:
        eng.slots_occupy_status[s] = True
    eng.slots_offsets.copy_(lens.to(device))
    eng.slots_prompt_len.copy_(lens.to(device))
    eng._offsets_host = [int(x) for x in lens]
    eng._prompt_host = [int(x) for x in lens]
    eng.slots_tokens.random_(0, cfg.vocab_size)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    launches0 = ops.launch_count()
    eng.decode_graphed(slots)                                # eager step (warms the kernels up)
    launches_per_step = ops.launch_count() - launches0
    eng.decode_graphed(slots)                                # captures, then replays
    for _ in range(max(args.warmup, 3)):
        eng.decode_graphed(slots)
    kv.check_status()
    model.check_status()
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    passes, host_ms, opened = [], [], []
    barrier()
    with sampler:
        for _ in range(max(1, args.reps)):
            e0.record()
            for _ in range(args.steps):
                eng.kv.wait_for_table_copies()               # (the device has started the previous step)
                t0 = time.perf_counter()
                eng.kv.prepare_step(slots)                   # (timed apart: the host share of a step)
                host_ms.append((time.perf_counter() - t0) * 1e3)
                opened.append(kv.pages_opened)
                eng._graph.replay()
                eng.kv.end_step()
            e1.record()
            barrier()
            passes.append(max_over_ranks(e0.elapsed_time(e1) / args.steps))
    ms_step = median(passes)
    # end to end: the serving loop needs the sampled tokens on the host every step (end-of-sequence test)
    host_tokens = torch.empty(B, dtype=torch.long).pin_memory()
    barrier()
    e0.record()
    for _ in range(args.steps):
        out = eng.decode_graphed(slots)
        host_tokens.copy_(out, non_blocking=False)
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    kv.check_status()
    model.check_status()
    # algorithmic attention bytes of a step on this rank (layer 0 dense, the others sparse)
    now = lens + args.warmup
    scored = (now - 4) // PAGE
    esz = 2
    b_sel = int(scored.sum()) * hkv * HEAD_DIM * esz
    b_dec = int((torch.clamp(scored, max=topk) + 2).sum()) * hkv * PAGE * HEAD_DIM * 2 * esz
    b_dense = int((scored + 2).sum()) * hkv * PAGE * HEAD_DIM * 2 * esz
    attn_bytes = (layers - 1) * (b_sel + b_dec) + b_dense
    weight_bytes = sum(t.numel() * 2 for L in model.layers for k, t in L.items() if t.dim() == 2) \
        + model.lm_head.numel() * 2
    if rank == 0:
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except Exception:
            pass
        peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
        ach = (attn_bytes + weight_bytes) / (ms_step * 1e-3) / 1e9
        emit({
            "metric": "block-top-k decode tokens/s (Qwen3-1.7B full-model step, 512 sequences, contexts in [512, 32768])",
            "value": B / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step,
            "ms_per_step_passes": {"reps": len(passes), "min": min(passes), "median": ms_step, "max": max(passes)},
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {wl['model']} full model, {layers} layers + final norm + "
                                   f"vocabulary projection + greedy sampling, {B} sequences, contexts uniform in "
                                   f"{[lo, hi]}, top-k {topk} pages, page {PAGE}, tensor parallel over {world} GPU(s)"
                                   + (f"; ONE RANK OF {shard_of} emulated, no exchange" if shard_of > 1 else ""),
                       "batch": B, "layers": layers, "topk_pages": topk, "parallelism": f"tp{world} by KV head",
                       "kv_pool_pages": pool_pages, "kv_bytes_per_layer_per_gpu": kv_bytes_layer,
                       "layers_share_one_physical_pool": alias,
                       "l2": "per-layer traffic exceeds the 126 MB L2"},
            "roofline": {"bound": "hbm", "kernel": "whole step (attention pages + summaries + weights)",
                         "achieved": ach, "peak": peak_gbs, "unit": "GB/s", "frac": ach / peak_gbs, "traffic": None,
                         "algorithmic_bytes": attn_bytes + weight_bytes, "attention_bytes": attn_bytes,
                         "weight_bytes": weight_bytes},
            "host": {"prepare_step_ms_median": median(host_ms), "prepare_step_ms_max": max(host_ms),
                     "table_bytes_per_step": kv.table_bytes, "pages_opened_first_step": opened[0],
                     "pages_opened_per_step_mean": sum(opened) / len(opened)},
            "e2e": {"value": B / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": kv.table_bytes, "d2h_bytes_per_step": B * 8,
                    "how": "Engine.decode_graphed + the sampled tokens copied to the host every step"},
            "cpu_baseline": None, "gpu_launches": launches_per_step * args.steps * max(1, args.reps),
            "gpu_launches_per_step": launches_per_step, "clocks": sampler.summary(),
        })
    if world > 1:
        # the captured step holds a collective of the process group (the ranks' local maxima of the vocabulary
        # projection): the graph has to be gone before the group is torn down
        torch.cuda.synchronize()
        eng._graph = None
        eng._graph_out = None
        out = None
        del eng, model, kv
        leave_group(dist, [])


def run_micro_exchange(args):
    """The NVLink exchange kernels alone on [batch, hidden] bf16 (under torchrun): every form, schedule and
    result, beside NCCL all-reduce (+ the add / norm kernel) and NCCL reduce-scatter."""
    import torch.distributed as dist
    import kinetics_b200 as kb
    from kinetics_b200 import _lib, ops
    from kinetics_b200.comm import FusedExchange

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    wl = dict(WORKLOADS[args.workload])
    rows = args.batch or wl["batch"]
    cols = kb.get_config(wl["model"]).hidden_size
    res = torch.randn(rows, cols, device=dev).to(torch.bfloat16)
    wb = torch.ones(cols, device=dev, dtype=torch.bfloat16)
    part = torch.randn(rows, cols, device=dev).to(torch.bfloat16)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    per_graph = 20                                           # calls captured into one CUDA graph: short
                                                             # exchanges are otherwise paced by the host's launches
    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(per_graph):
                fn()
        graph.replay()
        replays = max(1, args.steps // per_graph)
        dist.barrier(); torch.cuda.synchronize()
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / (replays * per_graph)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3                         # microseconds

    out = {"micro": "exchange", "ranks": world, "rows": rows, "cols": cols, "bytes": rows * cols * 2,
           "timing": "CUDA events around replays of a graph of 20 calls", "us": {}}
    forms = [("multicast", _lib.ALLREDUCE_MULTICAST)] + ([("peer", _lib.ALLREDUCE_PEER)] if world in (2, 4) else [])
    for fname, mode in forms:
        for schedule, result in (("lockstep", "allreduce_norm"), ("pipelined", "allreduce_norm"),
                                 ("pipelined", "allreduce"), ("pipelined", "scatter")):
            ex = FusedExchange(dist.group.WORLD, rows, cols, torch.bfloat16, dev, mode=mode, result=result,
                               schedule=schedule)
            ex.x.copy_(part)
            w = wb if result == "allreduce_norm" else None
            out["us"][f"{fname}/{schedule}/{result}"] = timed(lambda: ex(res, w, 1e-6))
            ops.raise_on_status(ex.status)
            del ex

    def nccl_allreduce_norm():
        dist.all_reduce(part)
        ops.add_rmsnorm(part, res, wb, 1e-6)

    mine = torch.empty(rows // world, cols, device=dev, dtype=torch.bfloat16)
    out["us"]["nccl all_reduce + add_rmsnorm kernel"] = timed(nccl_allreduce_norm)
    out["us"]["nccl all_reduce"] = timed(lambda: dist.all_reduce(part))
    out["us"]["nccl reduce_scatter"] = timed(lambda: dist.reduce_scatter_tensor(mine, part))
    if rank == 0:
        emit(out)
    leave_group(dist, [])


_RESULT_FD = None


def emit(line: dict) -> None:
    """The one JSON line of the run, on the process's original stdout."""
    text = json.dumps(line) + "\n"
    if _RESULT_FD is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text.encode())


def main():
    global _RESULT_FD
    args = parse()
    # Libraries print to stdout too (NCCL's version banner when NCCL_DEBUG is set): send everything
    # but the result line to stderr, so that stdout carries exactly one JSON line.
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.micro == "select":
        return run_micro_select(args)
    if args.micro == "exchange":
        return run_micro_exchange(args)
    if args.micro == "prefill":
        return run_micro_prefill(args)
    if args.impl == "reference":
        run_reference(args)
    elif WORKLOADS[args.workload].get("full_model"):
        run_full_model(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
