"""Import path twin of ``LiteSys/litesys/attention/sparsity_utils.py``: the dispatcher, the argument
normaliser and the block top-k mask (the only mask that is built; see ``cache_utils.py``)."""
from .cache_utils import attn_logits_processor, blockwise_topk_sparsity, preprocess_sparse_args  # noqa: F401

__all__ = ["attn_logits_processor", "blockwise_topk_sparsity", "preprocess_sparse_args"]
