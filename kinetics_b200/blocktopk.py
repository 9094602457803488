"""Command line of the block top-k layer benchmark: the flags and the printed summary of the
reference's ``benchmark/blocktopk.py:9-20,76-82``.

    python -m kinetics_b200.blocktopk --model Qwen/Qwen3-8B --gen_len 32768 --batch_size 256 \
        --page_size 16 --topk_page 64 --world_size 8

As in the reference, ``gen_len = 2N`` means a context of ``N`` tokens (``prefix_len = gen_len // 2``,
``benchmark/blocktopk.py:23``), one process stands for one of ``world_size`` tensor-parallel ranks and
the printed throughput is divided by ``world_size * num_hidden_layers`` (``:82``).  The model shape
comes from ``kinetics_b200.config`` (no download); ``forward`` is replayed from a CUDA graph instead of
``torch.compile``.
"""
from __future__ import annotations

import argparse
import time

import torch

from . import BlockTopkDecoderLayer, DecoderLayer, get_config, init_weights


def get_args(sparse: bool):
    parser = argparse.ArgumentParser()
    parser.add_argument("--model", type=str, required=True)
    parser.add_argument("--gen_len", type=int, default=32768)
    parser.add_argument("--page_size", type=int, default=16)
    if sparse:
        parser.add_argument("--topk_page", type=int, default=64)
    parser.add_argument("--batch_size", type=int, default=256)
    parser.add_argument("--repeat_time", type=int, default=256)
    parser.add_argument("--device", type=str, default="cuda")
    parser.add_argument("--dtype", type=str, default="bfloat16")
    parser.add_argument("--world_size", type=int, default=8)
    parser.add_argument("--warmup", type=int, default=200)
    return parser.parse_args()


def build_decoder_layer(config, args, sparse: bool):
    prefix_len = args.gen_len // 2
    max_len = prefix_len + 512
    dtype = getattr(torch, args.dtype)
    common = dict(config=config, world_size=args.world_size, batch_size=args.batch_size, prefix_len=prefix_len,
                  max_len=max_len, page_size=args.page_size, device=args.device, dtype=dtype)
    layer = BlockTopkDecoderLayer(topk_page=args.topk_page, **common) if sparse else DecoderLayer(**common)
    layer.apply(init_weights)
    layer.eval()
    layer.to(args.device, dtype=dtype)
    return layer


def run_benchmark(decoder_layer, hidden_states, repeat_time, warmup):
    static_in, _, graph = decoder_layer.make_graphed(hidden_states)
    for _ in range(warmup):
        static_in.copy_(hidden_states)
        graph.replay()
    torch.cuda.synchronize()
    start_time = time.time()
    for _ in range(repeat_time):
        static_in.copy_(hidden_states)          # the reference clones its input every iteration
        graph.replay()
    torch.cuda.synchronize()
    elapsed = time.time() - start_time
    return (repeat_time * hidden_states.size(0)) / elapsed


def main(sparse: bool = True):
    args = get_args(sparse)
    config = get_config(args.model)
    hidden_states = torch.randn(args.batch_size, 1, config.hidden_size, device=args.device,
                                dtype=getattr(torch, args.dtype))
    decoder_layer = build_decoder_layer(config, args, sparse)
    throughput = run_benchmark(decoder_layer, hidden_states, args.repeat_time, args.warmup)
    decoder_layer.check_status()
    print("\n=== Benchmark Summary ===")
    print(f"Model: {args.model.split('/')[-1]}")
    print(f"Prefix length: {args.gen_len // 2}")
    print(f"Page size: {args.page_size}")
    if sparse:
        print(f"Topk pages: {args.topk_page}")
    print(f"Batch size: {args.batch_size}")
    print(f"Throughput: {throughput / (args.world_size * config.num_hidden_layers):.2f} tokens/sec")


if __name__ == "__main__":
    main(True)
