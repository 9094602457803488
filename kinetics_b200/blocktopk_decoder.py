"""Import-compatible stand-in for the reference's ``benchmark/blocktopk_decoder.py``."""
from .layers import BlockTopkDecoderLayer, init_weights  # noqa: F401
