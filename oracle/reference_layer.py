"""The reference's decoder-layer forward on CPU tensors -- TEST / BASELINE INFRASTRUCTURE ONLY.

A torch restatement of ``BlockTopkDecoderLayer.forward`` (benchmark/blocktopk_decoder.py:186-240)
and of ``DecoderLayer.forward`` (benchmark/dense_decoder.py:191-234) that runs on host cores:
the four custom ops the reference routes to flashinfer are restated with plain torch statements
(the reference has no CPU implementation of them), everything else is the reference's own
sequence of torch calls.  It is what ``bench.py`` times as the CPU baseline and what the layer
test compares the CUDA layer with.  The product never imports it.

Uniform batch, as in the reference benchmark: every sequence has ``n`` full pages plus the page
being filled; ``page_table`` is ``[B, n+1]``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

P = 16


def rmsnorm(x, w, eps):
    """flashinfer.rmsnorm (benchmark/model_utils.py:12): fp32 statistics, result in x.dtype."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class ReferenceLayerCPU:
    """Weights + paged state of one layer shard on the host.

    `weights`: dict with wqkv.weight/bias, wo.weight, up/gate/down_proj.weight, the four norm weights.
    `kv_cache` [pages, 2, P, Hkv, D]; `summaries` [B, Hkv, n, D] (mean key per page) or None for dense.
    """

    def __init__(self, weights, kv_cache, page_table, summaries, num_heads, num_kv_heads, head_dim, eps, topk,
                 last_page_len=1):
        self.w = weights
        self.kv_cache, self.page_table, self.summaries = kv_cache, page_table.long(), summaries
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.eps, self.topk, self.last_page_len = eps, topk, last_page_len
        self.forced_pages = None      # [B, Hkv, m] physical pages to attend instead of the own selection

    def _append(self, k, v):
        # flashinfer.append_paged_kv_cache (benchmark/blocktopk_decoder.py:38-46): newest token
        # of sequence b goes to (last page of b, slot last_page_len - 1)
        page = self.page_table[:, -1]
        self.kv_cache[page, 0, self.last_page_len - 1] = k
        self.kv_cache[page, 1, self.last_page_len - 1] = v
        if self.summaries is not None and self.summaries.shape[2] > self.page_table.shape[1] - 1:
            filled = self.kv_cache[page, 0, : self.last_page_len].float()        # [B, c, Hkv, D]
            self.summaries[:, :, self.page_table.shape[1] - 1] = filled.mean(1).to(self.summaries.dtype)

    def _select(self, q):
        # benchmark/blocktopk_decoder.py:216-221, per kv head
        B = q.shape[0]
        G = self.num_heads // self.num_kv_heads
        n = self.page_table.shape[1] - 1
        qg = q.view(B, self.num_kv_heads, G, self.head_dim)
        csim = torch.einsum("b h g d, b h n d -> b h g n", qg, self.summaries[:, :, :n]).mean(dim=2)
        idx = torch.topk(csim, min(self.topk, n), dim=-1).indices                  # [B, Hkv, k]
        table = self.page_table[:, None, :].expand(B, self.num_kv_heads, n + 1)
        phys = torch.gather(table[:, :, :n], 2, idx)
        return torch.cat([phys, table[:, :, n:]], dim=-1)                          # [B, Hkv, k+1]

    def _attend(self, q, pages):
        # mylib::decode (benchmark/blocktopk_decoder.py:176-178): softmax(q K^T / sqrt(D)) V over the pages
        B = q.shape[0]
        G = self.num_heads // self.num_kv_heads
        kv = self.kv_cache[pages]                                                  # [B, Hkv, m, 2, P, Hkv, D]
        hsel = torch.arange(self.num_kv_heads)
        kv = kv[:, hsel, :, :, :, hsel]                                            # [Hkv, B, m, 2, P, D]
        kv = kv.permute(1, 0, 2, 3, 4, 5)
        m = pages.shape[-1]
        ntok = (m - 1) * P + self.last_page_len
        k = kv[:, :, :, 0].reshape(B, self.num_kv_heads, m * P, self.head_dim)[:, :, :ntok]
        v = kv[:, :, :, 1].reshape(B, self.num_kv_heads, m * P, self.head_dim)[:, :, :ntok]
        qg = q.view(B, self.num_kv_heads, G, self.head_dim)
        logits = torch.einsum("b h g d, b h s d -> b h g s", qg.float(), k.float()) / math.sqrt(self.head_dim)
        p = torch.softmax(logits, dim=-1)
        o = torch.einsum("b h g s, b h s d -> b h g d", p, v.float())
        return o.reshape(B, self.num_heads, self.head_dim).to(q.dtype)

    @torch.inference_mode()
    def forward(self, hidden_states):
        w = self.w
        residual = hidden_states
        hidden_states = rmsnorm(hidden_states, w["input_layernorm_weight"], self.eps)
        bsz, q_len, _ = hidden_states.size()
        q_dim, kv_dim = self.head_dim * self.num_heads, self.head_dim * self.num_kv_heads
        proj = F.linear(hidden_states, w["wqkv.weight"], w["wqkv.bias"])
        query_states, key_states, value_states = proj.split((q_dim, kv_dim, kv_dim), dim=-1)
        query_states = query_states.reshape(bsz, q_len, self.num_heads, self.head_dim)
        key_states = key_states.reshape(bsz, q_len, self.num_kv_heads, self.head_dim)
        value_states = value_states.reshape(bsz, self.num_kv_heads, self.head_dim)
        query_states = rmsnorm(query_states, w["qnorm_weight"], self.eps).reshape(bsz, self.num_heads, self.head_dim)
        key_states = rmsnorm(key_states, w["knorm_weight"], self.eps).reshape(bsz, self.num_kv_heads, self.head_dim)
        self._append(key_states, value_states)
        if self.forced_pages is not None:
            pages = self.forced_pages
        elif self.summaries is not None:
            pages = self._select(query_states)
        else:
            pages = self.page_table[:, None, :].expand(bsz, self.num_kv_heads, self.page_table.shape[1])
        self.last_q, self.last_pages = query_states, pages
        o = self._attend(query_states, pages).reshape(bsz, q_len, self.head_dim * self.num_heads)
        hidden_states = F.linear(o, w["wo.weight"])
        hidden_states = residual + hidden_states
        residual = hidden_states
        hidden_states = rmsnorm(hidden_states, w["post_attention_layernorm_weight"], self.eps)
        up = F.linear(hidden_states, w["up_proj.weight"])
        gate = F.linear(hidden_states, w["gate_proj.weight"])
        hidden_states = F.silu(gate) * up
        hidden_states = F.linear(hidden_states, w["down_proj.weight"])
        return residual + hidden_states
