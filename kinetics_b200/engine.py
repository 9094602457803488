"""Continuous-batching engine over a pooled paged KV cache.

Counterpart of ``LiteSys/litesys/engine/engine.py`` (the caller of the attention path): the same
slot-based loop -- prefill one request into a free slot, decode all occupied slots together, retire a
sequence on EOS / ``max_new_tokens`` / repetition and refill its slot (``engine.py:167-242``) -- the same
sampler (``:127-165``) and the same repetition check (``engine/utils.py:112-165``).  Two things differ:

* the KV cache is a pool of 16-token pages handed out by ``PagePool`` (``ktk_pool_*`` in the C ABI)
  instead of ``max_seq_len`` tokens reserved per slot (``batch_cache.py:32-40``), so admission is by
  free pages, and a request waits when the pool cannot promise ``prompt + max_new_tokens`` tokens;
* the model is whatever object has ``inference(input_ids, position_ids, batch_idx, kv) -> logits``
  (``models/qwen3.py:108-135`` in the reference); no model is part of this package.
"""
from __future__ import annotations

import copy
import ctypes
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from . import _lib, ops
from ._lib import check
from .batch_cache import PAGE, SINK, BatchKVManager


# --------------------------------------------------------------------------------------
# page pool (host side, C ABI)
# --------------------------------------------------------------------------------------

class PoolExhausted(RuntimeError):
    pass


class PagePool:
    """Which physical pages each sequence slot owns (``ktk_pool_*``).  Host-only bookkeeping."""

    def __init__(self, num_pages: int, max_slots: int, page_size: int = PAGE):
        self._lib = _lib.load()
        self._h = self._lib.ktk_pool_create(num_pages, max_slots, page_size)
        if not self._h:
            raise ValueError(self._lib.ktk_last_error().decode())
        self.num_pages, self.max_slots, self.page_size = num_pages, max_slots, page_size

    def close(self):
        if getattr(self, "_h", None):
            self._lib.ktk_pool_destroy(self._h)
            self._h = None

    __del__ = close

    @property
    def free_pages(self) -> int:
        return int(self._lib.ktk_pool_free_pages(self._h))

    def tokens(self, slot: int) -> int:
        return int(self._lib.ktk_pool_slot_tokens(self._h, slot))

    def pages(self, slot: int) -> int:
        return int(self._lib.ktk_pool_slot_pages(self._h, slot))

    def can_admit(self, max_total_tokens: int) -> bool:
        return (max_total_tokens + self.page_size - 1) // self.page_size <= self.free_pages

    def admit(self, slot: int, n_tokens: int, max_total_tokens: int) -> None:
        rc = self._lib.ktk_pool_admit(self._h, slot, n_tokens, max_total_tokens)
        if rc == _lib.KTK_ERR_TOO_LARGE:
            raise PoolExhausted(self._lib.ktk_last_error().decode())
        check(rc)

    def extend(self, slots: Sequence[int], tokens_each: int = 1) -> None:
        arr = (ctypes.c_int32 * len(slots))(*slots)
        rc = self._lib.ktk_pool_extend(self._h, arr, len(slots), tokens_each)
        if rc == _lib.KTK_ERR_TOO_LARGE:
            raise PoolExhausted(self._lib.ktk_last_error().decode())
        check(rc)

    def release(self, slot: int) -> None:
        check(self._lib.ktk_pool_release(self._h, slot))

    def export(self, slots: Sequence[int], pin: bool = False):
        """(kv_indices, kv_indptr, kv_last_page_len) as int32 CPU tensors for the slots, in that order."""
        n = len(slots)
        cap = sum(max(self.pages(s), 0) for s in slots)
        mk = (lambda *shape: torch.empty(*shape, dtype=torch.int32).pin_memory()) if pin else \
             (lambda *shape: torch.empty(*shape, dtype=torch.int32))
        indices, indptr, last = mk(max(cap, 1)), mk(n + 1), mk(max(n, 1))
        arr = (ctypes.c_int32 * n)(*slots)
        total = self._lib.ktk_pool_export(self._h, arr, n, ctypes.c_void_p(indices.data_ptr()), cap,
                                          ctypes.c_void_p(indptr.data_ptr()), ctypes.c_void_p(last.data_ptr()))
        if total < 0:
            check(int(total))
        return indices[:total], indptr, last[:n]


    def export_into(self, slots: Sequence[int], indices: torch.Tensor, indptr: torch.Tensor, last: torch.Tensor) -> int:
        """The same into caller-owned int32 CPU tensors (pinned ones, for a copy that overlaps); returns the
        number of page ids written."""
        n = len(slots)
        cached = getattr(self, "_export_slots", None)
        if cached is None or cached[0] != slots:           # the same batch step after step: build the C array once
            cached = (list(slots), (ctypes.c_int32 * n)(*slots))
            self._export_slots = cached
        arr = cached[1]
        total = self._lib.ktk_pool_export(self._h, arr, n, ctypes.c_void_p(indices.data_ptr()), indices.numel(),
                                          ctypes.c_void_p(indptr.data_ptr()), ctypes.c_void_p(last.data_ptr()))
        if total < 0:
            check(int(total))
        return int(total)


# --------------------------------------------------------------------------------------
# KV manager backed by the pool
# --------------------------------------------------------------------------------------

def _pool_tokens(length: int) -> int:
    """Tokens the pool has to hold for a sequence of `length` tokens: the sink page (4 tokens) takes a
    whole page, the pages behind it are ordinary 16-token pages (see batch_cache.py)."""
    if length <= 0:
        return 0
    return PAGE + max(length - SINK, 0)


class PooledKVManager(BatchKVManager):
    """``BatchKVManager`` whose pages come from a ``PagePool`` shared by all slots.

    Same attention surface (``compute_attention`` / ``decode`` / ``prefill_or_append`` /
    ``clear_cache``); in addition ``admit(slot, prompt_len, max_total_len)`` has to be called before a
    slot is first written (the engine does), and ``begin_step(slots)`` may be called with the active
    slots as a host list to spare the manager a device-to-host read of ``batch_idx``.
    """

    def __init__(self, config, max_batch_size: int, max_seq_len: int, device, dtype, num_pages: int,
                 alias_layers: bool = False, **kwargs):
        """`alias_layers`: every layer reads and writes ONE physical pool and one summary table (a benchmark
        device for models whose caches would not fit: the traffic per layer is real, the contents are not)."""
        self._num_pool_pages = int(num_pages)
        self._alias = bool(alias_layers)
        super().__init__(config, max_batch_size, max_seq_len, device, dtype, **kwargs)

    def _alloc_summaries(self):
        if not self._alias:
            return super()._alloc_summaries()
        one = torch.zeros(self.max_batch_size, self.num_key_value_heads, self.pages_per_slot, self.head_dim,
                          device=self.device, dtype=self.dtype)
        return [one] * self.num_layers

    # BatchKVManager allocates pages_per_slot * max_batch pages per layer; here the pool decides
    def _alloc_pages(self):
        total = self._num_pool_pages
        self.pool = PagePool(total, self.max_batch_size, PAGE)
        def pages():
            return torch.zeros(total, 2, PAGE, self.num_key_value_heads, self.head_dim, device=self.device,
                               dtype=self.dtype)
        self.kv_pages = [pages()] * self.num_layers if self._alias else [pages() for _ in range(self.num_layers)]
        self.kv_indices = None
        self._host_len = np.zeros((self.num_layers, self.max_batch_size), dtype=np.int64)
        self._active: Optional[List[int]] = None
        self._table_key = None
        self._table_val = None
        self._step_table = None          # set by prepare_step: the table every layer of the step uses
        self._step_offsets_advanced = False
        self._copies_done = None         # event behind the last step's table copies
        self._static = None              # static device buffers + pinned mirrors of that table

    # ---- admission / retirement
    def can_admit(self, max_total_len: int) -> bool:
        return self.pool.can_admit(_pool_tokens(max_total_len))

    def admit(self, slot: int, prompt_len: int, max_total_len: int) -> None:
        if max_total_len > self.max_length:
            raise ValueError(f"{max_total_len} tokens exceed max_seq_len {self.max_length}")
        self.pool.admit(slot, 0, _pool_tokens(max_total_len))

    def clear_cache(self, batch_idx: int):
        super().clear_cache(batch_idx)
        for i in range(self.num_layers):
            self._host_len[i][batch_idx] = 0
        if self.pool.tokens(batch_idx) >= 0:
            self.pool.release(batch_idx)
        self._table_key = None

    def begin_step(self, slots: Sequence[int]) -> None:
        self._active = list(slots)

    # ---- a decode step whose device work can sit in a CUDA graph
    def _static_buffers(self):
        if self._static is None:
            n, cap, dev = self.max_batch_size, self._num_pool_pages, self.device
            mk = lambda k: torch.empty(k, dtype=torch.int32)
            self._static = dict(
                h_indices=mk(cap).pin_memory(), h_indptr=mk(n + 1).pin_memory(), h_last=mk(n).pin_memory(),
                h_slot=mk(n).pin_memory(), h_order=mk(n).pin_memory(), d_indices=mk(cap).to(dev),
                d_indptr=mk(n + 1).to(dev), d_last=mk(n).to(dev), d_slot=mk(n).to(dev), d_order=mk(n).to(dev))
        return self._static

    def wait_for_table_copies(self) -> None:
        """The previous step's table copies read the pinned buffers when the stream reaches them: a host that
        runs ahead of the device must not overwrite them before that (the wait ends when the device has started
        the previous step, so host and device still overlap by one step)."""
        if self._copies_done is not None:
            self._copies_done.synchronize()

    def prepare_step(self, slots: Sequence[int]) -> None:
        """All the host work of one decode step over `slots` (every layer appends one token): the pool grows
        where a sequence crosses a page boundary, the CSR table goes into pinned memory and from there, with
        asynchronous copies on the current stream, into device buffers whose addresses never change -- so the
        device work that follows can be a replayed CUDA graph.  `end_step()` closes the step."""
        slots = list(slots)
        n = len(slots)
        st = self._static_buffers()
        self.wait_for_table_copies()
        idx = np.asarray(slots, dtype=np.int64)
        lengths = self._host_len[0, idx] + 1
        pool_tokens = lambda ln: np.where(ln > 0, PAGE + np.maximum(ln - SINK, 0), 0)
        grow = idx[pool_tokens(lengths) > pool_tokens(lengths - 1)]
        if grow.size:
            self.pool.extend(grow.tolist(), 1)
        total = self.pool.export_into(slots, st["h_indices"], st["h_indptr"], st["h_last"])
        st["h_last"].numpy()[:n] = np.where(lengths <= SINK, lengths, (lengths - SINK - 1) % PAGE + 1)
        st["h_slot"].numpy()[:n] = idx
        # rows of the batch from the longest to the shortest: the selection kernel's CTAs share them evenly
        st["h_order"].numpy()[:n] = np.argsort(-lengths, kind="stable")
        st["d_indices"][:total].copy_(st["h_indices"][:total], non_blocking=True)
        st["d_indptr"][:n + 1].copy_(st["h_indptr"][:n + 1], non_blocking=True)
        st["d_last"][:n].copy_(st["h_last"][:n], non_blocking=True)
        st["d_slot"][:n].copy_(st["h_slot"][:n], non_blocking=True)
        st["d_order"][:n].copy_(st["h_order"][:n], non_blocking=True)
        if self._copies_done is None:
            self._copies_done = torch.cuda.Event()
        self._copies_done.record()
        view = ops.PageView(SINK, self.local, None, st["d_slot"][:n], st["d_order"][:n])
        self._step_table = (st["d_indices"], st["d_indptr"][:n + 1], st["d_last"][:n], view)
        self._step_offsets_advanced = False
        self.kv_indices = st["d_indices"]
        self._host_len[:, idx] += 1
        self._active = slots
        self.table_bytes = 4 * (total + 4 * n + 1)
        # pages the step opened (a promise made at admission may already have reserved them)
        self.pages_opened = int(np.count_nonzero((lengths - SINK - 1) % PAGE == 0)) if n else 0

    def end_step(self) -> None:
        self._step_table = None
        self._table_key = None

    def assume_filled(self, lengths: dict, headroom: int = 0) -> None:
        """Benchmark set-up: slot -> number of tokens its pages are taken to hold already (the page contents
        are whatever the pool memory holds).  Admits the slots with a promise of `headroom` more tokens, grows
        them to that length, sets the lengths of every layer and rebuilds the page summaries from the pages."""
        slots = sorted(lengths)
        for s in slots:
            self.pool.admit(s, _pool_tokens(lengths[s]), _pool_tokens(min(lengths[s] + headroom, self.max_length)))
        lens_t = torch.zeros(self.max_batch_size, dtype=torch.int32)
        for s in slots:
            lens_t[s] = lengths[s]
        for layer in range(self.num_layers):
            self.kv_offset[layer].copy_(lens_t)
            for s in slots:
                self._host_len[layer][s] = lengths[s]
        indices, indptr, _ = self.pool.export(slots)
        last = torch.tensor([n if n <= SINK else (n - SINK - 1) % PAGE + 1 for n in (lengths[s] for s in slots)],
                            dtype=torch.int32)
        dev = self.device
        view = ops.PageView(SINK, self.local, None, torch.tensor(slots, dtype=torch.int32, device=dev))
        for layer in range(1 if self._alias else self.num_layers):
            ops.build_summaries(self.kv_pages[layer], self.summaries[layer], indices.to(dev), indptr.to(dev),
                                last.to(dev), status=self.status, view=view)

    # ---- page table of the active rows
    def _slots_of(self, batch_idx: torch.Tensor) -> List[int]:
        if self._active is not None and len(self._active) == batch_idx.numel():
            return self._active
        return [int(s) for s in batch_idx.tolist()]

    def _table_for(self, slots: List[int], lengths: List[int]):
        key = (tuple(slots), tuple(lengths))
        if key == self._table_key:
            return self._table_val
        grow = {}
        for s, n in zip(slots, lengths):
            have = self.pool.tokens(s)
            if have < 0:
                raise RuntimeError(f"slot {s} was not admitted to the page pool")
            d = _pool_tokens(n) - have
            if d > 0:
                grow.setdefault(d, []).append(s)
        for d, ss in grow.items():
            self.pool.extend(ss, d)
        indices, indptr, _ = self.pool.export(slots, pin=True)
        last = torch.tensor([n if n <= SINK else (n - SINK - 1) % PAGE + 1 for n in lengths], dtype=torch.int32)
        slot_t = torch.tensor(slots, dtype=torch.int32)
        dev = self.device
        val = (indices.to(dev, non_blocking=True), indptr.to(dev, non_blocking=True),
               last.to(dev, non_blocking=True), ops.PageView(SINK, self.local, None, slot_t.to(dev)))
        self._table_key, self._table_val = key, val
        return val

    def _table(self, batch_idx: torch.Tensor, lengths: torch.Tensor):
        raise RuntimeError("PooledKVManager builds its page table from host lengths (_table_for)")

    # ---- reference surface, on the pooled table
    def append_key_value_cache(self, new_key_cache, new_value_cache, batch_idx, layer_idx: int):
        if self._step_table is not None:
            # inside a prepared step: the table is in place and the host lengths are already advanced
            indices, indptr, last, view = self._step_table
            B = batch_idx.numel()
            k = new_key_cache.reshape(B, self.num_key_value_heads, self.head_dim).contiguous()
            v = new_value_cache.reshape(B, self.num_key_value_heads, self.head_dim).contiguous()
            ops.append_kv(k, v, self.kv_pages[layer_idx], self.summaries[layer_idx], indices, indptr, last,
                          status=self.status, view=view)
            if not self._step_offsets_advanced:
                # every layer appends one token in a prepared step: advance all layers' device lengths with
                # the first append (three small launches per step instead of three per layer)
                self._kv_offset_all[:, batch_idx] += 1
                self._step_offsets_advanced = True
            return indptr, last, view
        slots = self._slots_of(batch_idx)
        lengths = [int(self._host_len[layer_idx][s]) + 1 for s in slots]
        indices, indptr, last, view = self._table_for(slots, lengths)
        B = len(slots)
        k = new_key_cache.reshape(B, self.num_key_value_heads, self.head_dim).contiguous()
        v = new_value_cache.reshape(B, self.num_key_value_heads, self.head_dim).contiguous()
        ops.append_kv(k, v, self.kv_pages[layer_idx], self.summaries[layer_idx], indices, indptr, last,
                      status=self.status, view=view)
        for s in slots:
            self._host_len[layer_idx][s] += 1
        self.kv_offset[layer_idx][batch_idx] += 1
        self.kv_indices = indices
        return indptr, last, view

    def prefill_or_append(self, query_states, key_states, value_states, layer_idx, batch_idx):
        bsz, seq_len = query_states.shape[0], query_states.shape[2]
        assert bsz == 1, "prefill handles one sequence at a time, like the reference"
        slot = self._slots_of(batch_idx)[0]
        offset = int(self._host_len[layer_idx][slot])
        total = offset + seq_len
        indices, indptr, last, view = self._table_for([slot], [total])
        pages = self.kv_pages[layer_idx]
        append_indptr = torch.tensor([0, seq_len], device=self.device, dtype=torch.int32)
        ops.append_tokens(key_states[0].transpose(0, 1).to(self.dtype).contiguous(),
                          value_states[0].transpose(0, 1).to(self.dtype).contiguous(), append_indptr, pages,
                          self.summaries[layer_idx], indices, indptr, last, status=self.status, view=view)
        self._host_len[layer_idx][slot] = total
        self.kv_offset[layer_idx][slot] += seq_len
        q = query_states[0].transpose(0, 1).to(self.dtype).contiguous()          # [seq_len, Hq, D]
        out = ops.prefill_attention(q, append_indptr, seq_len, pages, indices, indptr, last, self.sm_scale,
                                    status=self.status, view=view)
        return out.reshape(bsz, seq_len, self.hidden_size)


# --------------------------------------------------------------------------------------
# sampler and repetition check
# --------------------------------------------------------------------------------------

def sample_next_tokens(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                       generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """logits [B, 1, V] -> tokens [B, 1] (engine.py:127-165): greedy below temperature 0.02, else top-k
    filter, softmax(logits / T), nucleus cut at top_p (the token that crosses it is kept), renormalise, draw."""
    if temperature < 0.02:
        return logits.argmax(dim=-1)
    logits = logits.squeeze(1)
    if top_k > 0:
        vals, idx = torch.topk(logits, top_k, dim=-1)
        logits = torch.full_like(logits, float("-inf")).scatter_(-1, idx, vals)
    probs = torch.softmax(logits / temperature, dim=-1)
    sorted_probs, sorted_idx = torch.sort(probs, descending=True, dim=-1)
    cum = torch.cumsum(sorted_probs, dim=-1)
    drop = cum > top_p
    drop[:, 1:] = drop[:, :-1].clone()
    drop[:, 0] = False
    sorted_probs = sorted_probs.masked_fill(drop, 0.0)
    sorted_probs = sorted_probs / sorted_probs.sum(dim=-1, keepdim=True)
    pick = torch.multinomial(sorted_probs, num_samples=1, generator=generator)
    return sorted_idx.gather(1, pick)


def recent_subseq_repeat_check(tokens: torch.Tensor, subseq_len: int = 10, recent_window: int = 100,
                               repeat_thresh: int = 4) -> bool:
    """True if the last `subseq_len` tokens occur at least `repeat_thresh` times among the
    `recent_window + subseq_len` tokens in front of them (engine/utils.py:112-165)."""
    n = tokens.numel()
    if n < subseq_len:
        return False
    window = tokens[max(0, n - recent_window - subseq_len): n - subseq_len]
    if window.numel() < subseq_len:
        return False
    recent = tokens[n - subseq_len:]
    hits = (window.unfold(0, subseq_len, 1) == recent).all(dim=-1)
    return int(hits.sum().item()) >= repeat_thresh


# --------------------------------------------------------------------------------------
# the engine loop
# --------------------------------------------------------------------------------------

class Engine:
    """Slot-based offline engine (``LLM`` in engine.py).  ``model`` has
    ``inference(input_ids [B, S], position_ids [B, S], batch_idx [B], kv) -> logits [B, S, V]``;
    ``kv`` is a ``BatchKVManager`` (every slot owns ``max_seq_len`` tokens) or a ``PooledKVManager``
    (admission by free pages)."""

    def __init__(self, model, kv, max_seq_len: int, device, top_p: float = 1.0, temperature: float = 0.0,
                 top_k: int = 0, eos: Sequence[int] = (151643, 151645), repeat_check: bool = True,
                 repeat_check_window: int = 1024, repeat_block_size: int = 64, seed: Optional[int] = None,
                 preprocess: Optional[Callable] = None, postprocess: Optional[Callable] = None):
        self.model, self.kv = model, kv
        self.device = torch.device(device)
        self.max_seq_len = max_seq_len
        self.max_batch_size = kv.max_batch_size
        self.top_p, self.top_k, self.temperature = top_p, top_k, temperature
        self.repeat_check = repeat_check
        self.repeat_block_size = repeat_block_size
        self.repeat_check_window = repeat_check_window
        self.repeat_thr = max((repeat_check_window // repeat_block_size) - 1, 2)
        self.eos_tensor = torch.tensor(list(eos), device=self.device)
        self.generator = None
        if seed is not None:
            self.generator = torch.Generator(device=self.device).manual_seed(seed)
        self.preprocess, self.postprocess = preprocess, postprocess
        n = self.max_batch_size
        self.slots_occupy_status = [False] * n
        self.slots_offsets = torch.zeros(n, dtype=torch.long, device=self.device)
        self.slots_prompt_len = torch.zeros(n, dtype=torch.long, device=self.device)
        self.slots_tokens = torch.zeros(n, max_seq_len, dtype=torch.long, device=self.device)
        self._offsets_host = [0] * n          # host mirrors: the loop below never reads lengths back
        self._prompt_host = [0] * n
        self.steps = 0

    # ---- per-slot operations (engine.py:85-125)
    def clear_request(self, slot: int) -> None:
        self.slots_occupy_status[slot] = False
        self.slots_offsets[slot] = 0
        self.slots_prompt_len[slot] = 0
        self.slots_tokens[slot].zero_()
        self._offsets_host[slot] = self._prompt_host[slot] = 0
        self.kv.clear_cache(slot)

    def can_admit(self, prompt_len: int, max_new_tokens: int) -> bool:
        total = prompt_len + max_new_tokens
        if total > self.max_seq_len:
            raise ValueError(f"prompt of {prompt_len} tokens + {max_new_tokens} new ones exceed max_seq_len")
        return self.kv.can_admit(total) if hasattr(self.kv, "can_admit") else True

    def prefill(self, slot: int, input_ids: torch.Tensor, max_new_tokens: int) -> None:
        seq_len = input_ids.shape[1]
        if hasattr(self.kv, "admit"):
            self.kv.admit(slot, seq_len, seq_len + max_new_tokens)
        input_ids = input_ids.to(self.device)
        position_ids = torch.arange(seq_len, dtype=torch.long, device=self.device).unsqueeze(0)
        self.slots_tokens[slot, :seq_len].copy_(input_ids[0])
        self.slots_offsets[slot] = seq_len
        self.slots_prompt_len[slot] = seq_len
        self._offsets_host[slot] = self._prompt_host[slot] = seq_len
        self.slots_occupy_status[slot] = True
        batch_idx = torch.tensor([slot], device=self.device)
        if hasattr(self.kv, "begin_step"):
            self.kv.begin_step([slot])
        if self.temperature < 0.02 and hasattr(self.model, "next_tokens"):
            self.slots_tokens[slot, seq_len] = self.model.next_tokens(input_ids, position_ids, batch_idx, self.kv,
                                                                      last_only=True)[-1]
        else:
            logits = self.model.inference(input_ids, position_ids, batch_idx, self.kv)[:, -1:, :]
            self.slots_tokens[slot, seq_len] = self._sample(logits).reshape(())

    def decode(self, slots: List[int]) -> torch.Tensor:
        batch_idx = torch.tensor(slots, device=self.device)
        offset = self.slots_offsets[batch_idx].unsqueeze(1)
        input_ids = self.slots_tokens[batch_idx].gather(dim=-1, index=offset)
        if hasattr(self.kv, "begin_step"):
            self.kv.begin_step(slots)
        if self.temperature < 0.02 and hasattr(self.model, "next_tokens"):
            next_tokens = self.model.next_tokens(input_ids, offset, batch_idx, self.kv)      # greedy, see _decode_device
        else:
            next_tokens = self._sample(self.model.inference(input_ids, offset, batch_idx, self.kv))
        self.slots_offsets[batch_idx] += 1
        for s in slots:
            self._offsets_host[s] += 1
        # the new token goes behind the one just consumed (copy_new_tokens, engine/utils.py:33-47)
        self.slots_tokens[batch_idx, self.slots_offsets[batch_idx]] = next_tokens.reshape(-1)
        self.steps += 1
        return (next_tokens.reshape(-1, 1) == self.eos_tensor.view(1, -1)).any(dim=1)

    # ---- the same step with its device work replayed from a CUDA graph
    def _decode_device(self, batch_idx: torch.Tensor):
        pos = self.slots_offsets[batch_idx]
        input_ids = self.slots_tokens[batch_idx, pos].unsqueeze(1)
        if self.temperature < 0.02 and hasattr(self.model, "next_tokens"):
            # greedy: the model may find the token without materialising (or, across ranks, gathering) the logits
            next_tokens = self.model.next_tokens(input_ids, pos.unsqueeze(1), batch_idx, self.kv).reshape(-1)
        else:
            logits = self.model.inference(input_ids, pos.unsqueeze(1), batch_idx, self.kv)
            next_tokens = self._sample(logits).reshape(-1)
        self.slots_offsets[batch_idx] += 1
        self.slots_tokens[batch_idx, pos + 1] = next_tokens
        return next_tokens

    def decode_graphed(self, slots: List[int]) -> torch.Tensor:
        """`decode` for a `PooledKVManager` and greedy sampling, with everything the device does in one step --
        embedding, all layers, vocabulary projection, argmax, token bookkeeping -- captured once and replayed.
        The host part of a step is `kv.prepare_step` (page growth + table export into static buffers).  The set
        of slots must not change between calls (capture a new engine step otherwise).  Returns the sampled
        tokens [len(slots)] (a device tensor the next replay overwrites)."""
        if self.temperature >= 0.02:
            raise ValueError("decode_graphed samples greedily (temperature < 0.02)")
        slots = list(slots)
        if getattr(self, "_graph_slots", None) != slots:
            self._graph_slots, self._graph = slots, None
            self._graph_batch_idx = torch.tensor(slots, device=self.device)
        self.kv.prepare_step(slots)
        if self._graph is None:
            # one eager pass warms every kernel up (and is this call's step); the graph serves the later calls
            self._graph_out = self._decode_device(self._graph_batch_idx)
            torch.cuda.synchronize(self.device)
            self.kv.end_step()
            self._graph = False
        elif self._graph is False:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._graph_out = self._decode_device(self._graph_batch_idx)
            # capture does not execute: run the captured step now
            graph.replay()
            self._graph = graph
            self.kv.end_step()
        else:
            self._graph.replay()
            self.kv.end_step()
        for s in slots:
            self._offsets_host[s] += 1
        self.steps += 1
        return self._graph_out

    def _sample(self, logits: torch.Tensor) -> torch.Tensor:
        return sample_next_tokens(logits, self.temperature, self.top_k, self.top_p, self.generator)

    # ---- the loop (engine.py:167-242)
    def offline_exec(self, requests: list, max_new_tokens: int) -> list:
        done, pending = [], 0
        total = len(requests)
        gen_counts = [0] * self.max_batch_size
        meta = [None] * self.max_batch_size

        preprocessed = -1                          # index of the last request the hook has seen

        def try_fill(slot: int) -> bool:
            nonlocal pending, preprocessed
            if pending >= total:
                return False
            req = requests[pending]
            if self.preprocess is not None and preprocessed < pending:
                # once per request, as in the reference: a request that has to wait for pages comes back
                # here on every refill attempt, and a hook need not be idempotent
                self.preprocess(req)
                preprocessed = pending
            ids = torch.as_tensor(req["input_ids"]).reshape(1, -1)
            if not self.can_admit(ids.shape[1], max_new_tokens):
                return False                       # the pool is full: wait for a sequence to retire
            self.prefill(slot, ids, max_new_tokens)
            gen_counts[slot] = 1
            meta[slot] = req
            pending += 1
            return True

        for slot in range(self.max_batch_size):
            if not try_fill(slot):
                break
        if pending == 0 and total > 0:
            raise PoolExhausted("the first request does not fit the page pool")

        while any(self.slots_occupy_status):
            active = [i for i, on in enumerate(self.slots_occupy_status) if on]
            is_eos = self.decode(active).tolist()
            for i, slot in enumerate(active):
                gen_counts[slot] += 1
                seq_len, prompt_len = self._offsets_host[slot], self._prompt_host[slot]
                is_repeat = False
                if self.repeat_check and seq_len > self.repeat_check_window:
                    is_repeat = recent_subseq_repeat_check(
                        self.slots_tokens[slot, prompt_len:seq_len], subseq_len=self.repeat_block_size,
                        recent_window=self.repeat_check_window, repeat_thresh=self.repeat_thr)
                if not (is_eos[i] or gen_counts[slot] >= max_new_tokens or is_repeat):
                    continue
                track_back = self.repeat_block_size if is_repeat else 0
                result = copy.deepcopy(meta[slot])
                result["output_tokens"] = self.slots_tokens[slot, prompt_len:seq_len - track_back].tolist()
                if self.postprocess is not None:
                    self.postprocess(result)
                done.append(result)
                self.clear_request(slot)
                meta[slot] = None
            # refill every free slot the pool can serve (a retired sequence may have freed enough pages
            # for a request that had to wait)
            for slot in range(self.max_batch_size):
                if not self.slots_occupy_status[slot] and not try_fill(slot):
                    break
            if pending < total and not any(self.slots_occupy_status):
                raise PoolExhausted("a request does not fit the empty page pool")
        return done
