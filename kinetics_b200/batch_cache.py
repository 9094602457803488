"""KV manager with the interface of LiteSys ``BatchKVManager`` on the paged block top-k kernels.

Counterpart of ``LiteSys/litesys/attention/batch_cache.py:10-168``: same constructor
(``config, max_batch_size, max_seq_len, device, dtype, **sparse_kwargs``), same methods
(``compute_attention``, ``append_key_value_cache``, ``prefill_or_append``, ``decode``,
``clear_cache``) and the same results as the reference's decode chain
``copy_to_cache -> qk -> attn_logits_processor -> softmax -> sv`` (``batch_cache.py:154-168``,
``cache_utils.py``, ``sparsity_utils.py``), but without ever materialising the dense
``[B, Hq, max_len]`` logits the reference writes and masks:

* K/V live in 16-token pages; logical page 0 of a slot holds the 4 sink tokens, page ``p >= 1``
  the tokens ``[4 + 16(p-1), 4 + 16p)``, so pages coincide with the reference's block grid
  (``sparsity_utils.py:33-37``: blocks start behind the sink);
* the append also maintains the mean key of every page (the block mean of ``:37`` moved in front
  of the dot product);
* with ``attn_block_topk`` set, a decode step scores the blocks that lie more than ``attn_local``
  tokens behind the end, keeps the top-k of them plus the sink and everything after them, and
  attends only those pages (``blockwise_topk_sparsity``, ``:24-47``); layers in
  ``attn_layer_skip`` (default ``[0]``, ``:211``) and sequences with too few blocks stay dense
  (``:27-32``).

Lengths are kept per SLOT and looked up through ``batch_idx``; the reference's kernels read the
offset of the active-batch ROW instead (``cache_utils.py:67,106,149``), which is only right while
the active slots are ``0..n-1``.

Built: the block top-k mask (``attn_block_topk``), the token top-k mask (``attn_topk``,
``sparsity_utils.py:6-21``: every key is read for the logits, only the kept tokens' values after the
mask) and the dense path.  The strided, random and local-only masks of ``sparsity_utils.py`` raise
``NotImplementedError`` here.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import ops

SINK = 4          # sparsity_utils.py:24 (`sink=4`, never overridden by the dispatcher)
PAGE = ops.PAGE_SIZE


def preprocess_sparse_args(**kwargs):
    """Same normalisation and checks as sparsity_utils.py:198-213."""
    attn_topk = kwargs.get("attn_topk", None)
    attn_local = kwargs.get("attn_local", None)
    attn_block_topk = kwargs.get("attn_block_topk", None)
    attn_random_select = kwargs.get("attn_random_select", None)
    attn_random_nsample = kwargs.get("attn_random_nsample", None)
    n = sum(x is not None for x in (attn_topk, attn_block_topk, attn_random_select, attn_random_nsample))
    assert n <= 1, "Only one of the sparsity parameters can be provided"
    if n:
        assert attn_local is not None, "attn_local must be provided if use_nonlocal_sparsity is True"
    kwargs["use_nonlocal_sparsity"] = n
    kwargs["use_sparsity"] = n + (attn_local is not None)
    kwargs["attn_layer_skip"] = kwargs.get("attn_layer_skip", [0])
    return kwargs


class BatchKVManager:
    def __init__(self, config, max_batch_size: int, max_seq_len: int, device, dtype, **kwargs):
        self.config = config
        self.max_length = max_seq_len
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_batch_size = max_batch_size
        self.head_dim = getattr(config, "head_dim", config.hidden_size // config.num_attention_heads)
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            self.world_size = torch.distributed.get_world_size()
        else:
            self.world_size = 1
        self.num_layers = config.num_hidden_layers
        self.hidden_size = self.head_dim * config.num_attention_heads // self.world_size
        self.num_key_value_heads = config.num_key_value_heads // self.world_size
        self.num_attention_heads = config.num_attention_heads // self.world_size
        self.num_key_value_groups = config.num_attention_heads // config.num_key_value_heads
        self.sparse_kwargs = preprocess_sparse_args(**kwargs)
        if self.head_dim != ops.HEAD_DIM:
            raise ValueError(f"only head_dim={ops.HEAD_DIM} is built")

        sk = self.sparse_kwargs
        self.block_topk: Optional[int] = sk.get("attn_block_topk", None)
        self.token_topk: Optional[int] = sk.get("attn_topk", None)
        self.local = int(sk.get("attn_local") or 0)
        if sk["use_sparsity"] and self.block_topk is None and self.token_topk is None:
            raise NotImplementedError("only attn_block_topk, attn_topk (+ attn_local) and dense attention are built; "
                                      "random and local-only masks are not")
        if self.block_topk is not None:
            if sk.get("attn_block_size", PAGE) != PAGE or sk.get("attn_stride", None) is not None:
                raise NotImplementedError(f"attn_block_size must be {PAGE} and attn_stride unset")
        self.layer_skip = list(sk["attn_layer_skip"])

        self.pages_per_slot = 1 + (max(max_seq_len - SINK, 0) + PAGE - 1) // PAGE
        self._alloc_pages()
        self.summaries = self._alloc_summaries()
        # one [layers, max_batch] tensor; kv_offset[layer] (the reference's list) are its rows
        self._kv_offset_all = torch.zeros(self.num_layers, max_batch_size, device=self.device, dtype=torch.int32)
        self.kv_offset = list(self._kv_offset_all.unbind(0))
        self.status = ops.new_status(self.device)
        self.row_width = ops.PageView(SINK, self.local).row_width(self.block_topk) if self.block_topk else 0
        self._sel = None
        self._workspace = None
        self._logits = None          # fp32 [max_batch, Hq, max_len], token-level top-k only (the reference's attn_score)
        self.sm_scale = 1.0 / math.sqrt(self.head_dim)

    # ------------------------------------------------------------------ page bookkeeping
    def _alloc_pages(self):
        """Slot b owns physical pages [b * P_max, (b + 1) * P_max); the table is the identity."""
        total = self.pages_per_slot * self.max_batch_size
        self.kv_pages = [torch.zeros(total, 2, PAGE, self.num_key_value_heads, self.head_dim, device=self.device,
                                     dtype=self.dtype) for _ in range(self.num_layers)]
        self.kv_indices = torch.arange(total, device=self.device, dtype=torch.int32)

    def _alloc_summaries(self):
        """One mean-key row per (slot, kv head, logical page) and layer."""
        return [torch.zeros(self.max_batch_size, self.num_key_value_heads, self.pages_per_slot, self.head_dim,
                            device=self.device, dtype=self.dtype) for _ in range(self.num_layers)]

    def _table(self, batch_idx: torch.Tensor, lengths: torch.Tensor):
        """Per active row: start of its page list, page count, tokens in its last page, view."""
        slot = batch_idx.to(torch.int32).contiguous()
        lengths = lengths.to(torch.int32)
        behind = torch.clamp(lengths - SINK, min=0)
        count = torch.where(lengths > 0, 1 + (behind + PAGE - 1) // PAGE, torch.zeros_like(lengths))
        last = torch.where(lengths > SINK, (behind - 1) % PAGE + 1, lengths)
        start = slot * self.pages_per_slot
        view = ops.PageView(SINK, self.local, count.to(torch.int32).contiguous(), slot)
        return start.contiguous(), last.to(torch.int32).contiguous(), view

    def _ws(self, B: int, entries: int):
        splits = ops.decode_num_splits(B, self.num_key_value_heads, self.num_key_value_groups, entries, self.dtype)
        need = ops.decode_workspace_bytes(B, self.num_key_value_heads, self.num_key_value_groups, splits)
        if need and (self._workspace is None or self._workspace.numel() < need):
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        return splits

    # ------------------------------------------------------------------ reference surface
    def append_key_value_cache(self, new_key_cache, new_value_cache, batch_idx, layer_idx: int):
        """batch_cache.py:76-84: one token per active sequence; advances kv_offset."""
        lengths = self.kv_offset[layer_idx][batch_idx] + 1
        start, last, view = self._table(batch_idx, lengths)
        B = batch_idx.numel()
        k = new_key_cache.reshape(B, self.num_key_value_heads, self.head_dim).contiguous()
        v = new_value_cache.reshape(B, self.num_key_value_heads, self.head_dim).contiguous()
        ops.append_kv(k, v, self.kv_pages[layer_idx], self.summaries[layer_idx], self.kv_indices, start, last,
                      status=self.status, view=view)
        self.kv_offset[layer_idx][batch_idx] += 1
        return start, last, view

    def compute_attention(self, query_states, key_states, value_states, layer_idx, batch_idx):
        """batch_cache.py:86-110: q [B, Hq, S, D], k/v [B, Hkv, S, D] -> [B, S, Hq * D]."""
        bsz, seq_len = query_states.shape[0], query_states.shape[2]
        if seq_len > 1:
            return self.prefill_or_append(query_states, key_states, value_states, layer_idx, batch_idx)
        output = self.decode(query_states, key_states, value_states, batch_idx, layer_idx)
        return output.reshape(bsz, seq_len, self.hidden_size)

    def decode(self, query, key, value, batch_idx, layer_idx):
        """batch_cache.py:154-168 in three launches: append, select, attend."""
        start, last, view = self.append_key_value_cache(key, value, batch_idx, layer_idx)
        B = batch_idx.numel()
        q = query.reshape(B, self.num_attention_heads, self.head_dim).contiguous()
        pages = self.kv_pages[layer_idx]
        sparse = self.block_topk is not None and layer_idx not in self.layer_skip
        if self.token_topk is not None and layer_idx not in self.layer_skip:
            return self._decode_token_topk(q, pages, start, last, view, batch_idx, layer_idx)
        if sparse:
            if self._sel is None or self._sel.shape[0] < B:
                self._sel = torch.empty(self.max_batch_size, self.num_key_value_heads, self.row_width,
                                        dtype=torch.int32, device=self.device)
            sel = self._sel[:B]
            ops.select_pages(q, self.summaries[layer_idx], self.kv_indices, start, last, self.block_topk,
                             pages.shape[0], out=sel, status=self.status, view=view)
            splits = self._ws(B, self.row_width)
            return ops.sparse_decode(q, pages, sel, start, last, self.sm_scale, self._workspace, splits,
                                     status=self.status, view=view, topk=self.block_topk)
        splits = self._ws(B, self.pages_per_slot)
        return ops.dense_decode(q, pages, self.kv_indices, start, last, self.pages_per_slot, self.sm_scale,
                                self._workspace, splits, status=self.status, view=view)

    def _decode_token_topk(self, q, pages, start, last, view, batch_idx, layer_idx):
        """attn_topk (sparsity_utils.py:6-21): the reference's own chain qk -> mask -> softmax -> sv
        (batch_cache.py:154-168) on the paged cache.  Every key is read (the mask needs every logit), of the
        values only those of the kept tokens."""
        B = q.shape[0]
        if self._logits is None:
            width = (self.max_length + 127) // 128 * 128
            self._logits = torch.empty(self.max_batch_size, self.num_attention_heads, width, dtype=torch.float32,
                                       device=self.device)
        logits = self._logits[:B]
        lengths = self.kv_offset[layer_idx][batch_idx].to(torch.int32).contiguous()
        ops.paged_qk(q, pages, self.kv_indices, start, last, logits, self.sm_scale, status=self.status, view=view)
        ops.token_topk_mask(logits, lengths, self.num_attention_heads, self.num_key_value_heads, self.token_topk,
                            self.local, SINK, status=self.status)
        ops.softmax_rows(logits, lengths)
        return ops.paged_sv(logits, B, pages, self.kv_indices, start, last, status=self.status, view=view)

    def prefill_or_append(self, query_states, key_states, value_states, layer_idx, batch_idx):
        """batch_cache.py:112-145: one sequence, seq_len tokens appended behind what the slot holds, causal
        attention over the whole slot -- two launches: the chunk goes into its pages (summaries of the touched
        pages refreshed), then the prefill kernel reads the slot's pages through the table."""
        bsz, seq_len = query_states.shape[0], query_states.shape[2]
        assert bsz == 1, "prefill handles one sequence at a time, like the reference"
        slot = int(batch_idx.item())
        offset = int(self.kv_offset[layer_idx][slot].item())
        pages = self.kv_pages[layer_idx]
        self.kv_offset[layer_idx][slot] += seq_len
        total = offset + seq_len
        bi = torch.tensor([slot], device=self.device, dtype=torch.int64)
        start, last, view = self._table(bi, torch.tensor([total], device=self.device, dtype=torch.int32))
        append_indptr = torch.tensor([0, seq_len], device=self.device, dtype=torch.int32)
        ops.append_tokens(key_states[0].transpose(0, 1).to(self.dtype).contiguous(),
                          value_states[0].transpose(0, 1).to(self.dtype).contiguous(), append_indptr, pages,
                          self.summaries[layer_idx], self.kv_indices, start, last, status=self.status, view=view)
        q = query_states[0].transpose(0, 1).to(self.dtype).contiguous()          # [seq_len, Hq, D]
        out = ops.prefill_attention(q, append_indptr, seq_len, pages, self.kv_indices, start, last, self.sm_scale,
                                    status=self.status, view=view)
        return out.reshape(bsz, seq_len, self.hidden_size)

    def clear_cache(self, batch_idx: int):
        """batch_cache.py:147-152.  Pages behind a slot's length are never read, so only the lengths
        (and the summaries, for tidiness) are reset."""
        for i in range(self.num_layers):
            self.kv_offset[i][batch_idx].zero_()
            self.summaries[i][batch_idx].zero_()

    def check_status(self):
        ops.raise_on_status(self.status)
