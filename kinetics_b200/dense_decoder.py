"""Import-compatible stand-in for the reference's ``benchmark/dense_decoder.py``."""
from .layers import DecoderLayer, init_weights  # noqa: F401
