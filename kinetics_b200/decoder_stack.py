"""A stack of decoder layers with random weights: the caller a full-model decode step needs.

The layer loop of ``LiteSys/litesys/models/qwen3.py:89-143`` (``layer_compute`` + ``inference``) and, with a
process group, of ``qwen3_dist.py:87-122`` (two all-reduces per layer), written over this library's ops:
fused q/k-norm + rotary embedding, ``kv.compute_attention`` (block top-k paged decode, or the prefill kernel),
residual add + RMSNorm in one kernel, and -- across ranks -- the NVLink exchange kernels, where the down_proj
all-reduce of layer i is fused with the residual add and the INPUT norm of layer i+1.

It has ``inference(input_ids, position_ids, batch_idx, kv)`` like the reference's models, so ``Engine`` drives
it.  Weights are drawn from N(0, 0.02) (no checkpoint is read): this is a benchmark and test vehicle, not a
model loader.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import ops, tp


def merge_rank_maxima(every: torch.Tensor) -> torch.Tensor:
    """every [ranks, rows, 2] fp32 = each rank's (largest logit, its token id) per row -> the token of the overall
    largest logit per row; among equal maxima the lowest token id (what an argmax over the whole row gives)."""
    best = every[:, :, 0].max(dim=0).values
    ids = torch.where(every[:, :, 0] == best, every[:, :, 1], torch.full_like(best, float("inf")))
    return ids.min(dim=0).values.long()


class DecoderStack:
    def __init__(self, config, device, dtype=torch.bfloat16, process_group=None, max_positions: int = 40960,
                 decode_batch: int = 0, seed: int = 0, num_layers: Optional[int] = None,
                 logits_dtype=torch.float32, shard_vocab: bool = False):
        # logits_dtype: fp32 as the reference returns them (qwen3.py:141); None leaves them in the compute dtype,
        # which greedy sampling can take as they are (the argmax of bf16 logits is the argmax of their fp32 copies)
        self.logits_dtype = logits_dtype
        # shard_vocab (with a process group): every rank keeps vocab_size / world rows of the vocabulary projection;
        # `next_tokens` then finds the greedy token from the ranks' local maxima (a few KB exchanged) instead of
        # every rank multiplying with the whole matrix.  `inference` needs the whole matrix and refuses.
        self.shard_vocab = bool(shard_vocab)
        self.config, self.device, self.dtype = config, torch.device(device), dtype
        self.group = process_group
        self.world = torch.distributed.get_world_size(process_group) if process_group is not None else 1
        self.rank = torch.distributed.get_rank(process_group) if process_group is not None else 0
        self.hidden = config.hidden_size
        self.head_dim = config.head_dim
        self.num_heads = config.num_attention_heads // self.world
        self.num_kv_heads = config.num_key_value_heads // self.world
        self.eps = config.rms_norm_eps
        self.num_layers = num_layers if num_layers is not None else config.num_hidden_layers
        H, D, Hq, Hkv, inter = self.hidden, self.head_dim, config.num_attention_heads, config.num_key_value_heads, \
            config.intermediate_size
        g = torch.Generator(device=self.device).manual_seed(seed)      # the same full-size weights on every rank

        def w(*shape):
            return torch.empty(*shape, device=self.device, dtype=dtype).normal_(0.0, 0.02, generator=g)

        self.embed_tokens = w(config.vocab_size, H)
        self.lm_head = w(config.vocab_size, H)
        self.vocab_lo = 0
        self.norm_weight = torch.ones(H, device=self.device, dtype=dtype)
        self.layers = []
        for _ in range(self.num_layers):
            wqkv, wo = w((Hq + 2 * Hkv) * D, H), w(H, Hq * D)
            up, gate, down = w(inter, H), w(inter, H), w(H, inter)
            if self.world > 1:
                wqkv, _ = tp.shard_wqkv(wqkv, None, Hq, Hkv, D, self.rank, self.world)
                wo = tp.shard_wo(wo, Hq, D, self.rank, self.world)
                up, gate, down = tp.shard_mlp(up, gate, down, self.rank, self.world)
            # gate_proj and up_proj as one stacked weight: one GEMM, whose halves the activation kernel reads
            self.layers.append(dict(
                wqkv=wqkv, wo=wo, gate_up=torch.cat((gate, up), dim=0).contiguous(), down=down,
                qnorm=torch.ones(D, device=self.device, dtype=dtype), knorm=torch.ones(D, device=self.device, dtype=dtype),
                input_norm=torch.ones(H, device=self.device, dtype=dtype),
                post_norm=torch.ones(H, device=self.device, dtype=dtype)))
        # rotary tables (qwen3.py:48-60; attention_scaling is 1 for the default rope)
        inv_freq = 1.0 / (config.rope_theta ** (torch.arange(0, D, 2, device=self.device).float() / D))
        freqs = torch.outer(torch.arange(max_positions, device=self.device).float(), inv_freq)
        emb = torch.cat((freqs, freqs), dim=-1)
        self.cos_cache, self.sin_cache = emb.cos().to(dtype).contiguous(), emb.sin().to(dtype).contiguous()
        # the two exchanges of a decode step, shared by all layers (they run one after the other)
        self.ex_o = self.ex_d = None
        if self.world > 1 and decode_batch > 0:
            from .comm import FusedExchange
            self.ex_o = FusedExchange(process_group, decode_batch, H, dtype, self.device, result="allreduce_norm")
            self.ex_d = FusedExchange(process_group, decode_batch, H, dtype, self.device, result="allreduce_norm")
        self.decode_batch = decode_batch
        if self.shard_vocab and self.world > 1:
            if config.vocab_size % self.world:
                raise ValueError(f"vocab_size {config.vocab_size} does not divide over {self.world} ranks")
            rows = config.vocab_size // self.world
            self.vocab_lo = self.rank * rows
            self.lm_head = self.lm_head[self.vocab_lo:self.vocab_lo + rows].clone()

    # -- the sum over ranks of a partial GEMM output, + residual, + RMSNorm with `weight`
    def _reduce_add_norm(self, ex, a, b_t, residual, weight):
        rows = a.shape[0]
        if self.world == 1:
            return ops.add_rmsnorm(torch.mm(a, b_t), residual, weight, self.eps)
        if ex is not None and rows == self.decode_batch:
            torch.mm(a, b_t, out=ex.x)
            return ex(residual.contiguous(), weight, self.eps)
        part = torch.mm(a, b_t)                                        # prefill rows: NCCL, then the add + norm kernel
        torch.distributed.all_reduce(part, group=self.group)
        return ops.add_rmsnorm(part, residual, weight, self.eps)

    @torch.no_grad()
    def inference(self, input_ids, position_ids, batch_idx, kv):
        if self.shard_vocab and self.world > 1:
            raise RuntimeError("inference() returns full logits: build the stack without shard_vocab, or call next_tokens()")
        bsz, seq_len = input_ids.shape
        n = self._hidden(input_ids, position_ids, batch_idx, kv)
        # n is the final RMSNorm of the residual stream (qwen3.py:139)
        logits = torch.mm(n, self.lm_head.t())
        if self.logits_dtype is not None:
            logits = logits.to(self.logits_dtype)
        return logits.view(bsz, seq_len, -1)

    @torch.no_grad()
    def next_tokens(self, input_ids, position_ids, batch_idx, kv, last_only: bool = False):
        """Greedy tokens [rows] of a decode step (the argmax of the logits `inference` would return; among equal
        maxima the lowest token id); last_only: only the token behind the last row (a prompt).  With shard_vocab
        every rank multiplies with its rows of the vocabulary projection only and the ranks exchange
        (maximum, token id) pairs."""
        n = self._hidden(input_ids, position_ids, batch_idx, kv)
        if last_only:
            n = n[-1:]
        logits = torch.mm(n, self.lm_head.t())                         # [rows, vocab or vocab / world]
        if not (self.shard_vocab and self.world > 1):
            return logits.argmax(dim=-1)
        vals, idx = logits.max(dim=-1)
        pair = torch.stack((vals.float(), (idx + self.vocab_lo).float()), dim=1)       # ids < 2^24: exact in fp32
        every = torch.empty(self.world, *pair.shape, device=pair.device, dtype=pair.dtype)
        torch.distributed.all_gather_into_tensor(every, pair, group=self.group)
        return merge_rank_maxima(every)

    def _hidden(self, input_ids, position_ids, batch_idx, kv):
        """The layer loop: the final RMSNorm of the residual stream, [rows, hidden]."""
        bsz, seq_len = input_ids.shape
        assert bsz == 1 or seq_len == 1, f"Operation Not Supported with input shape {tuple(input_ids.shape)}"
        rows = bsz * seq_len
        x = F.embedding(input_ids.reshape(-1), self.embed_tokens)                      # [rows, H] residual stream
        pos = position_ids.reshape(-1)
        _, n = ops.add_rmsnorm(x, None, self.layers[0]["input_norm"], self.eps)
        for i, L in enumerate(self.layers):
            proj = torch.mm(n, L["wqkv"].t())
            q, k, v = ops.qkv_norm(proj, L["qnorm"], L["knorm"], self.eps, self.num_heads, self.num_kv_heads,
                                   self.cos_cache, self.sin_cache, pos)
            # [rows, heads, D] -> [bsz, heads, seq_len, D], the layout compute_attention takes
            shape = lambda t, h: t.view(bsz, seq_len, h, self.head_dim).transpose(1, 2)
            attn = kv.compute_attention(shape(q, self.num_heads), shape(k, self.num_kv_heads),
                                        shape(v, self.num_kv_heads), i, batch_idx)
            attn = attn.reshape(rows, self.num_heads * self.head_dim)
            x, n = self._reduce_add_norm(self.ex_o, attn, L["wo"].t(), x, L["post_norm"])
            gu = torch.mm(n, L["gate_up"].t())
            half = gu.shape[1] // 2
            act = ops.silu_mul(gu[:, :half], gu[:, half:])
            nxt = self.layers[i + 1]["input_norm"] if i + 1 < self.num_layers else self.norm_weight
            x, n = self._reduce_add_norm(self.ex_d, act, L["down"].t(), x, nxt)
        return n

    def check_status(self):
        for ex in (self.ex_o, self.ex_d):
            if ex is not None:
                ops.raise_on_status(ex.status)
