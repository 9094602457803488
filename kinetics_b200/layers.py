"""Decoder layers with block top-k / dense paged decode attention.

Drop-in counterparts of the reference's ``BlockTopkDecoderLayer``
(benchmark/blocktopk_decoder.py:96-265) and ``DecoderLayer`` (benchmark/dense_decoder.py:94-234):
same constructor arguments, ``forward(hidden_states[B, 1, H]) -> [B, 1, H]`` and
``prepare_wrapper``.  Differences, all on purpose:

* the paged append, page selection and attention run hand-written CUDA kernels (libktk.so)
  instead of flashinfer / ATen; the linear layers stay cuBLAS;
* ``compressed_key_cache`` holds the mean key of every page (maintained by the append), not
  random numbers (reference :166-168), for every local kv head (the reference asserts one, :165);
* the selection computed in ``forward`` is the one the attention consumes (the reference rebinds
  ``self.topk_page_indices`` at :221 while flashinfer keeps the buffer from :157);
* ``last_kv_lens`` starts at 1 (the token the step appends) instead of 0 (:149);
* the torch ops are registered once at import, so dense and sparse layers share a process;
* with ``process_group`` set, the o_proj and the down_proj partial sums are reduced over the ranks
  (LiteSys litesys/models/qwen3_dist.py:111-112 and :120-121) and the residual is added once; the
  reference benchmark only divides head counts.  ``down_exchange="scatter"`` leaves rank r with the rows
  [r*B/N, (r+1)*B/N) of the layer output (a reduce-scatter) instead of all rows on every rank.
"""
from __future__ import annotations

import contextlib
import math
import weakref
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops


def init_weights(m):
    """Same initialisation as benchmark/blocktopk_decoder.py:88-94."""
    if isinstance(m, nn.Linear):
        nn.init.kaiming_uniform_(m.weight, a=math.sqrt(5))
        if m.bias is not None:
            fan_in, _ = nn.init._calculate_fan_in_and_fan_out(m.weight)
            bound = 1 / math.sqrt(fan_in)
            nn.init.uniform_(m.bias, -bound, bound)


def interleaved_page_table(batch_size: int, pages_per_req: int, device) -> torch.Tensor:
    """[B, pages_per_req] with entry [b, p] = p * B + b (benchmark/blocktopk_decoder.py:141)."""
    p = torch.arange(pages_per_req, dtype=torch.int32, device=device) * batch_size
    return (p[None, :] + torch.arange(batch_size, dtype=torch.int32, device=device)[:, None]).contiguous()


def random_page_table(batch_size: int, pages_per_req: int, num_pages: int, device, seed: int) -> torch.Tensor:
    """[B, pages_per_req] drawn from one global random permutation of the physical pages."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g)[: batch_size * pages_per_req]
    return perm.to(torch.int32).view(batch_size, pages_per_req).to(device).contiguous()


class _EventPair:
    """Brackets a kernel with CUDA events on the current stream when timing is switched on."""

    def __init__(self, sink, name):
        self.sink, self.name = sink, name

    def __enter__(self):
        if self.sink is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()

    def __exit__(self, *exc):
        if self.sink is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.sink.setdefault(self.name, []).append((self.start, end))
        return False


class _PagedDecoderLayer(nn.Module):
    """Shared body: weights, paged KV state, the non-attention part of forward."""

    def __init__(self, config, world_size, batch_size, prefix_len, max_len, page_size, device, dtype,
                 page_table: str = "interleaved", process_group=None, seed: int = 0, variant: int = 0,
                 kv_cache: Optional[torch.Tensor] = None, context_lens=None, fused_allreduce: bool = False,
                 down_exchange: str = "allreduce", exchange_schedule: Optional[str] = None):
        super().__init__()
        self.num_heads = config.num_attention_heads // world_size
        self.num_kv_heads = config.num_key_value_heads // world_size
        self.num_key_value_groups = self.num_heads // self.num_kv_heads
        self.head_dim = config.head_dim
        self.dim = config.hidden_size
        self.intermediate_size = config.intermediate_size // world_size
        self.max_position_embeddings = config.max_position_embeddings
        self.rope_theta = getattr(config, "rope_theta", 1e6)
        eos = getattr(config, "eos_token_id", None)
        self.eos_tokens = eos if isinstance(eos, list) else [eos]
        self.hidden_act = getattr(config, "hidden_act", "silu")
        self.ffn_frac = getattr(config, "ffn_frac", 1.0)

        eps = config.rms_norm_eps
        self.qnorm_weight = nn.Parameter(torch.ones(self.head_dim))
        self.qnorm_variance_epsilon = eps
        self.knorm_weight = nn.Parameter(torch.ones(self.head_dim))
        self.knorm_variance_epsilon = eps
        self.input_layernorm_weight = nn.Parameter(torch.ones(self.dim))
        self.input_layernorm_variance_epsilon = eps
        self.post_attention_layernorm_weight = nn.Parameter(torch.ones(self.dim))
        self.post_attention_layernorm_variance_epsilon = eps

        total_head_dim = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        self.wqkv = nn.Linear(self.dim, total_head_dim, bias=True)
        self.wo = nn.Linear(self.head_dim * self.num_heads, self.dim, bias=False)
        self.up_proj = nn.Linear(self.dim, self.intermediate_size, bias=False)
        self.gate_proj = nn.Linear(self.dim, self.intermediate_size, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size, self.dim, bias=False)

        self.batch_size = batch_size
        self.prefix_len = prefix_len
        self.page_size = page_size
        self.device = device
        self.dtype = dtype
        self.process_group = process_group
        self.variant = variant
        # with a process group: sum the o_proj and down_proj partials either with NCCL followed by the
        # add (+ norm) kernel, or (fused_allreduce) with the exchange kernels of comm.py
        if down_exchange not in ("allreduce", "scatter"):
            raise ValueError("down_exchange: 'allreduce' or 'scatter'")
        self.down_exchange = down_exchange
        self.fused = self.fused_down = None
        if process_group is not None and fused_allreduce:
            from .comm import FusedExchange
            self.fused = FusedExchange(process_group, batch_size, self.dim, dtype, device,
                                       result="allreduce_norm", schedule=exchange_schedule)
            self.fused_down = FusedExchange(process_group, batch_size, self.dim, dtype, device,
                                            result=down_exchange)
        if page_size != ops.PAGE_SIZE or self.head_dim != ops.HEAD_DIM:
            raise ValueError(f"only page_size={ops.PAGE_SIZE}, head_dim={ops.HEAD_DIM} are built")

        # paged KV state: prefix fills num_pages_per_req pages, the step appends into one more.
        # `context_lens` (one prefix length per sequence) makes the batch ragged: sequence b then owns
        # context_lens[b] // page_size full pages plus the page the step writes into (which already holds
        # context_lens[b] % page_size tokens; a multiple of the page size means the step opens a new
        # page), laid out as one CSR list over a randomly permuted ("fragmented") or packed page pool.
        self.max_num_pages = max_num_pages = max_len // page_size
        self.total_pages = max_num_pages * batch_size
        if context_lens is None:
            self.num_pages_per_req = n = prefix_len // page_size
            if n + 1 > max_num_pages:
                raise ValueError("max_len leaves no page for the decoded token")
            if page_table == "interleaved":
                table = interleaved_page_table(batch_size, n + 1, device)
            elif page_table == "random":
                table = random_page_table(batch_size, n + 1, self.total_pages, device, seed)
            else:
                raise ValueError(f"page_table {page_table!r}: 'interleaved' or 'random'")
            self.page_table = table                                  # [B, n+1]
            self.paged_kv_indices = table.view(-1)
            self.full_kv_indptr = (torch.arange(batch_size + 1, dtype=torch.int32, device=device) * (n + 1))
            self.max_pages_per_seq = n + 1
        else:
            lens = torch.as_tensor(context_lens, dtype=torch.int64)
            if lens.numel() != batch_size or int(lens.min()) < 0 or int(lens.max()) // page_size + 1 > max_num_pages:
                raise ValueError("context_lens: one length per sequence, each leaving a page for the new token")
            counts = lens // page_size + 1
            self.num_pages_per_req = int(counts.max()) - 1
            self.max_pages_per_seq = int(counts.max())
            indptr = torch.zeros(batch_size + 1, dtype=torch.int64)
            indptr[1:] = torch.cumsum(counts, 0)
            total_used = int(indptr[-1])
            if page_table == "random":
                g = torch.Generator(device="cpu").manual_seed(seed)
                ids = torch.randperm(self.total_pages, generator=g)[:total_used]
            else:
                ids = torch.arange(total_used)
            self.page_table = None
            self.paged_kv_indices = ids.to(torch.int32).to(device).contiguous()
            self.full_kv_indptr = indptr.to(torch.int32).to(device)
        self.context_lens = context_lens
        if context_lens is None:
            self.last_kv_lens = torch.ones(batch_size, dtype=torch.int32, device=device)
        else:
            self.last_kv_lens = (lens % page_size + 1).to(torch.int32).to(device)
        self.qkv_indptr = torch.arange(batch_size + 1, dtype=torch.int32, device=device)
        self.status = ops.new_status(device)

        shape = (self.total_pages, 2, page_size, self.num_kv_heads, self.head_dim)
        if kv_cache is None:
            kv_cache = torch.randn(*shape, dtype=dtype, device=device)
        elif tuple(kv_cache.shape) != shape or kv_cache.dtype != dtype:
            raise ValueError(f"kv_cache must be {shape} {dtype}")
        self.kv_cache = kv_cache          # may be shared with another layer (dense next to sparse)
        # the bindings ops.py keeps per cache address go when the layer goes
        weakref.finalize(self, ops.unbind_address, kv_cache.data_ptr())
        self.decode_run = torch.ops.mylib.decode
        self.capture = None               # set to a dict to keep q / k / v of the last forward (tests)
        self.timers = None                # set to a dict name -> list of (start, end) CUDA events

    # -- attention-specific parts, provided by the subclasses --
    def _attention(self, query_states):
        raise NotImplementedError

    def _bind(self):
        raise NotImplementedError

    def _mlp(self, hidden_states, residual):
        """SwiGLU MLP.  One rank: the residual add rides in the epilogue of the down projection GEMM.
        Several ranks: the down_proj partials are summed over the ranks and the residual is added once
        (litesys/models/qwen3_dist.py:120-122)."""
        up = self.up_proj(hidden_states)
        gate = self.gate_proj(hidden_states)
        if self.hidden_act == "silu":
            hidden_states = torch.ops.ktk.silu_mul(gate, up)
        else:
            from transformers.activations import ACT2FN
            hidden_states = ACT2FN[self.hidden_act](gate) * up
        if self.process_group is None:
            return torch.addmm(residual, hidden_states, self.down_proj.weight.t())
        if self.fused_down is not None:
            torch.mm(hidden_states, self.down_proj.weight.t(), out=self.fused_down.x)
            with self._timed("exchange_down_proj"):
                out, _ = self.fused_down(residual.contiguous())
            return out
        part = torch.mm(hidden_states, self.down_proj.weight.t())
        with self._timed("exchange_down_proj"):
            if self.down_exchange == "scatter":
                world = torch.distributed.get_world_size(self.process_group)
                rank = torch.distributed.get_rank(self.process_group)
                per = part.shape[0] // world
                out = torch.empty(per, part.shape[1], dtype=part.dtype, device=part.device)
                torch.distributed.reduce_scatter_tensor(out, part, group=self.process_group)
                return out.add_(residual[rank * per:(rank + 1) * per])
            torch.distributed.all_reduce(part, group=self.process_group)
            return part.add_(residual)

    @torch.no_grad()      # the reference uses inference_mode (:186); torch 2.11 cannot compile a function decorated with it
    def forward(self, hidden_states):
        # The torch ops find this layer's page state through its kv_cache.  Under torch.compile the binding
        # made by prepare_wrapper() stands (the reference calls it right after compiling, blocktopk.py:41-44).
        if not torch.compiler.is_compiling():
            self._bind()
        bsz, q_len, _ = hidden_states.size()
        residual = hidden_states.reshape(bsz * q_len, self.dim)
        # input RMSNorm (mylib::layer_norm of the reference, :192), 16-byte accesses
        hidden_states = torch.ops.ktk.rms_norm(residual, self.input_layernorm_weight,
                                               self.input_layernorm_variance_epsilon)
        proj = self.wqkv(hidden_states)
        # split + q-norm + k-norm (:198-207) in one launch
        query_states, key_states, value_states = torch.ops.ktk.qkv_norm(
            proj, self.qnorm_weight, self.knorm_weight, self.qnorm_variance_epsilon, self.num_heads,
            self.num_kv_heads)
        if self.capture is not None:
            self.capture.update(q=query_states.clone(), k=key_states.clone(), v=value_states.clone())
        with self._timed("append"):
            torch.ops.mylib.update_kv(key_states, value_states, self.qkv_indptr, self.kv_cache,
                                      self.paged_kv_indices, self.full_kv_indptr, self.last_kv_lens)
        o = self._attention(query_states)
        if self.capture is not None:
            self.capture.update(o=o.clone())
        o = o.reshape(bsz * q_len, self.head_dim * self.num_heads)
        if self.fused is not None:
            # o_proj partial straight into the symmetric buffer, then all-reduce + residual add + norm at once
            torch.mm(o, self.wo.weight.t(), out=self.fused.x)
            with self._timed("exchange_o_proj"):
                residual, hidden_states = self.fused(residual.contiguous(), self.post_attention_layernorm_weight,
                                                     self.post_attention_layernorm_variance_epsilon)
        else:
            hidden_states = self.wo(o)
            if self.process_group is not None:
                with self._timed("exchange_o_proj"):
                    torch.distributed.all_reduce(hidden_states, group=self.process_group)
            # residual add + post-attention RMSNorm (:229-231) in one pass
            residual, hidden_states = torch.ops.ktk.add_rms_norm(hidden_states, residual,
                                                                 self.post_attention_layernorm_weight,
                                                                 self.post_attention_layernorm_variance_epsilon)
        # [B, 1, H]; under down_exchange="scatter" the [B / world, 1, H] rows this rank owns
        return self._mlp(hidden_states, residual).view(-1, q_len, self.dim)

    def _timed(self, name):
        return contextlib.nullcontext() if self.timers is None else _EventPair(self.timers, name)

    def check_status(self):
        """Synchronising check of the device status words: the layer's own and those of its exchanges
        (an expired cross-rank wait shows up here)."""
        ops.raise_on_status(self.status)
        for ex in (self.fused, self.fused_down):
            if ex is not None:
                ops.raise_on_status(ex.status)

    def make_graphed(self, example: torch.Tensor, warmup: int = 3, static_in: Optional[torch.Tensor] = None):
        """Capture one forward in a CUDA graph.  Returns (static_input, static_output, graph).  `static_in`:
        the buffer the graph reads its input from (default: a copy of `example`)."""
        if static_in is None:
            static_in = example.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.forward(static_in)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = self.forward(static_in)
        return static_in, static_out, graph


class BlockTopkDecoderLayer(_PagedDecoderLayer):
    """benchmark/blocktopk_decoder.py:96 -- block top-k sparse decode attention."""

    def __init__(self, config, world_size, batch_size, prefix_len, max_len, page_size, topk_page, device, dtype,
                 **kw):
        super().__init__(config, world_size, batch_size, prefix_len, max_len, page_size, device, dtype, **kw)
        self.topk_page = topk_page
        n = self.num_pages_per_req
        self.topk_page_indices = torch.full((batch_size * self.num_kv_heads * (topk_page + 1),), -1,
                                            dtype=torch.int32, device=device)
        # one summary row per (sequence, kv head, logical page); reference: [B, n, D] for one head
        self.compressed_key_cache = torch.zeros(batch_size, self.num_kv_heads, self.max_pages_per_seq + 7, self.head_dim,
                                                dtype=dtype, device=device)
        self.rebuild_summaries()
        ops.bind_summaries(self.kv_cache, self.compressed_key_cache)
        self.prepare_wrapper(prefix_len)

    def rebuild_summaries(self):
        ops.build_summaries(self.kv_cache, self.compressed_key_cache, self.paged_kv_indices, self.full_kv_indptr,
                            self.last_kv_lens, status=self.status)

    def _sel_view(self):
        return self.topk_page_indices.view(self.batch_size, self.num_kv_heads, self.topk_page + 1)

    def _attention(self, query_states):
        # benchmark/blocktopk_decoder.py:216-221, one kernel
        with self._timed("select"):
            torch.ops.ktk.select_pages_into(query_states, self.compressed_key_cache, self.paged_kv_indices,
                                            self.full_kv_indptr, self.last_kv_lens, self.topk_page, self.total_pages,
                                            self._sel_view(), self.status)
        with self._timed("decode"):
            return self.decode_run(query_states, self.kv_cache)

    def _bind(self):
        ops.bind_summaries(self.kv_cache, self.compressed_key_cache)
        ops.bind_decode_plan(self.decode_plan)

    def prepare_wrapper(self, prefix_len=None, topk_page_indices=None):
        """Bind the decode plan (reference: flashinfer wrapper.plan, :243-265).

        `topk_page_indices`, if given, pre-loads the selection buffer ([B * Hkv * (topk+1)] int32
        physical pages); forward overwrites it with its own selection.
        """
        if topk_page_indices is not None:
            self.topk_page_indices.copy_(topk_page_indices.view(-1).to(torch.int32))
        plan = ops.DecodePlan(self.kv_cache, self.full_kv_indptr, self.last_kv_lens, sel_pages=self._sel_view(),
                              sm_scale=1.0 / math.sqrt(self.head_dim), variant=self.variant, status=self.status)
        ops.bind_decode_plan(plan)
        self.decode_plan = plan


class DecoderLayer(_PagedDecoderLayer):
    """benchmark/dense_decoder.py:94 -- dense paged decode attention over every page."""

    def __init__(self, config, world_size, batch_size, prefix_len, max_len, page_size, device, dtype, **kw):
        super().__init__(config, world_size, batch_size, prefix_len, max_len, page_size, device, dtype, **kw)
        self.prepare_wrapper()

    def _attention(self, query_states):
        with self._timed("decode"):
            return self.decode_run(query_states, self.kv_cache)

    def _bind(self):
        ops.bind_decode_plan(self.decode_plan)

    def prepare_wrapper(self):
        plan = ops.DecodePlan(self.kv_cache, self.full_kv_indptr, self.last_kv_lens,
                              kv_indices=self.paged_kv_indices, max_pages_per_seq=self.max_pages_per_seq,
                              sm_scale=1.0 / math.sqrt(self.head_dim), variant=self.variant, status=self.status)
        ops.bind_decode_plan(plan)
        self.decode_plan = plan
