"""Command line of the dense paged decode benchmark (reference: ``benchmark/dense.py``).

    python -m kinetics_b200.dense --model Qwen/Qwen3-8B --gen_len 32768 --batch_size 256 --page_size 16 --world_size 8
"""
from .blocktopk import main

if __name__ == "__main__":
    main(False)
