"""kinetics_b200 -- block top-k sparse decode attention over a paged KV cache, for B200 (sm_100a).

The package mirrors the operator surface of Infini-AI-Lab/Kinetics for this one path
(``benchmark/blocktopk_decoder.py``, ``benchmark/dense_decoder.py``, ``LiteSys/litesys/attention``)
on top of hand-written CUDA kernels in ``libktk.so`` (C ABI: ``include/ktk.h``).
Importing the package loads the library; if it has not been built the import fails.
"""
from . import _lib

_lib.load()   # no fallback: a missing library is an ImportError

from . import ops  # noqa: E402  (registers the torch ops)
from .config import LayerConfig, get_config  # noqa: E402
from .layers import BlockTopkDecoderLayer, DecoderLayer, init_weights  # noqa: E402
from .batch_cache import BatchKVManager  # noqa: E402
from .engine import Engine, PagePool, PooledKVManager, PoolExhausted  # noqa: E402
from .decoder_stack import DecoderStack  # noqa: E402

__all__ = ["ops", "LayerConfig", "get_config", "BlockTopkDecoderLayer", "DecoderLayer", "init_weights",
           "BatchKVManager", "DecoderStack", "Engine", "PagePool", "PooledKVManager", "PoolExhausted"]
