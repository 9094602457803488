"""The one exchange of the tensor-parallel layer -- the sum of the ranks' o_proj partial outputs
(LiteSys/litesys/models/qwen3_dist.py:111-112) -- fused with the residual add and the
post-attention RMSNorm that follow it (:113-114), in one hand-written kernel over NVLink
(``ktk_allreduce_add_rmsnorm``): with plain peer loads and stores at 2 and 4 ranks, through NVSwitch
multicast above.

PyTorch provides the plumbing only: buffers that every rank can reach and that are mapped into one
multicast object (``torch.distributed._symmetric_memory``); the reduction (``multimem.ld_reduce`` or
peer loads), the arithmetic, the stores to every rank and the cross-rank flag waits are in
``csrc/ktk_comm.cu``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib, ops
from ._lib import check


class FusedAllReduceNorm:
    """Owns the symmetric buffers of one layer: `x` (the o_proj GEMM writes its partial output here),
    `sum` (what the kernel multicasts back to every rank) and the local `norm`."""

    def __init__(self, group, rows: int, cols: int, dtype, device, mode: int = _lib.ALLREDUCE_AUTO):
        import torch.distributed._symmetric_memory as symm_mem

        if dtype != torch.bfloat16:
            raise TypeError("the fused all-reduce is built for bfloat16")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.rows, self.cols, self.mode = rows, cols, mode
        lib = _lib.load()
        self.grid = int(lib.ktk_allreduce_grid(rows, self.world))
        if rows % self.world or self.grid <= 0:
            raise ValueError(f"{rows} rows do not divide over {self.world} ranks")
        self.x = symm_mem.empty(rows, cols, dtype=dtype, device=device)
        self.sum = symm_mem.empty(rows, cols, dtype=dtype, device=device)
        self.norm = torch.empty(rows, cols, dtype=dtype, device=device)
        self.flags = symm_mem.empty(self.grid * self.world, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.launch_count = torch.zeros(self.grid, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._hx = symm_mem.rendezvous(self.x, group)
        self._hs = symm_mem.rendezvous(self.sum, group)
        self._hf = symm_mem.rendezvous(self.flags, group)
        peer_form = mode == _lib.ALLREDUCE_PEER or (mode == _lib.ALLREDUCE_AUTO and self.world in (2, 4))
        for h in (self._hx, self._hs):
            if not peer_form and not h.multicast_ptr:
                raise RuntimeError("this system gives no NVSwitch multicast mapping: use the NCCL all-reduce")
        torch.cuda.synchronize(device)
        self._hf.barrier()          # every rank's flags are zero before anybody signals

    def __call__(self, residual: torch.Tensor, weight: torch.Tensor, eps: float):
        """`self.x` holds this rank's partial output.  Returns (residual + sum over ranks, its RMSNorm)."""
        if residual.shape != self.x.shape or residual.dtype != self.x.dtype or not residual.is_contiguous():
            raise ValueError("residual must match the symmetric buffer")
        check(_lib.load().ktk_allreduce_add_rmsnorm(
            ctypes.c_void_p(self._hx.multicast_ptr or None), ctypes.c_void_p(self._hx.buffer_ptrs_dev),
            ctypes.c_void_p(residual.data_ptr()), ctypes.c_void_p(weight.data_ptr()),
            ctypes.c_void_p(self._hs.multicast_ptr or None), ctypes.c_void_p(self._hs.buffer_ptrs_dev),
            ctypes.c_void_p(self.sum.data_ptr()), ctypes.c_void_p(self.norm.data_ptr()),
            ctypes.c_void_p(self._hf.buffer_ptrs_dev),
            ctypes.c_void_p(self.launch_count.data_ptr()), self.rank, self.world, self.rows, self.cols, eps,
            self.mode, ctypes.c_void_p(self.status.data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        ops._launched()
        return self.sum, self.norm
