"""The two exchanges of the tensor-parallel layer -- the sums of the ranks' o_proj and down_proj partial
outputs (LiteSys/litesys/models/qwen3_dist.py:111-112 and :120-121) -- each fused with what follows it
(residual add, RMSNorm) in one hand-written kernel over NVLink: plain peer loads and stores at 2 and
4 ranks, NVSwitch multicast (``multimem``) above.

PyTorch provides the plumbing only: buffers that every rank can reach and that are mapped into one
multicast object (``torch.distributed._symmetric_memory``); the reduction (``multimem.ld_reduce`` or
peer loads), the arithmetic, the stores to every rank and the cross-rank flag waits are in
``csrc/ktk_exchange.cu`` (row-pipelined schedule) and ``csrc/ktk_comm.cu`` (lock-step schedule).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib, ops
from ._lib import check

RESULTS = {"allreduce_norm": _lib.EXCHANGE_ALLREDUCE_NORM, "allreduce": _lib.EXCHANGE_ALLREDUCE,
           "scatter": _lib.EXCHANGE_SCATTER}


class FusedExchange:
    """Owns the symmetric buffers of one exchange.

    ``x``     [rows, cols], the GEMM writes this rank's partial output here
    ``sum``   all-reduce results: residual + sum over ranks, all rows, on every rank;
              ``scatter``: [rows / world, cols], the rows this rank owns (``row_range``)
    ``norm``  ``allreduce_norm`` only: RMSNorm of ``sum``

    ``schedule``: "pipelined" (ktk_exchange_rows) or "lockstep" (ktk_allreduce_add_rmsnorm, the
    all-reduce + norm result only); None picks by size for the all-reduce + norm.
    """

    PIPELINED_UP_TO = 8 << 20          # bytes of [rows, cols] bf16 up to which the all-reduce + norm is pipelined

    def __init__(self, group, rows: int, cols: int, dtype, device, mode: int = _lib.ALLREDUCE_AUTO,
                 result: str = "allreduce_norm", schedule: str = None):
        import torch.distributed._symmetric_memory as symm_mem

        if schedule is None:
            # all-reduce + norm, measured inside CUDA graphs on four B200s: up to 8 MiB the row-pipelined kernel
            # is ahead (2 MiB: 20 us against 28 us, 8 MiB: 40 against 47 -- no closing barrier before the norm of
            # the peers' rows); from 16 MiB the lock-step one is (32 MiB: 105 against 120 -- one system-scope
            # release per CTA instead of one per row).  Only the pipelined kernel has the other two results.
            small = rows * cols * 2 <= self.PIPELINED_UP_TO
            schedule = "pipelined" if result != "allreduce_norm" or small else "lockstep"

        if dtype != torch.bfloat16:
            raise TypeError("the fused exchange is built for bfloat16")
        if result not in RESULTS:
            raise ValueError(f"result {result!r}: one of {sorted(RESULTS)}")
        if schedule not in ("pipelined", "lockstep") or (schedule == "lockstep" and result != "allreduce_norm"):
            raise ValueError("schedule: 'pipelined', or 'lockstep' for the all-reduce + norm result")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.rows, self.cols, self.mode, self.result, self.schedule = rows, cols, mode, result, schedule
        lib = _lib.load()
        grid_fn = lib.ktk_exchange_grid if schedule == "pipelined" else lib.ktk_allreduce_grid
        self.grid = int(grid_fn(rows, self.world))
        if rows % self.world or self.grid <= 0:
            raise ValueError(f"{rows} rows do not divide over {self.world} ranks")
        per = rows // self.world
        self.row_range = (self.rank * per, (self.rank + 1) * per)
        self.x = symm_mem.empty(rows, cols, dtype=dtype, device=device)
        self.norm = None
        if result == "scatter":
            self.sum = torch.empty(per, cols, dtype=dtype, device=device)
            # the kernel addresses its output by global row: hand it where row 0 would be
            self._out_ptr = self.sum.data_ptr() - self.row_range[0] * cols * self.sum.element_size()
        else:
            self.sum = symm_mem.empty(rows, cols, dtype=dtype, device=device)
            self._out_ptr = self.sum.data_ptr()
            if result == "allreduce_norm":
                self.norm = torch.empty(rows, cols, dtype=dtype, device=device)
        self.flags = symm_mem.empty(self.grid * self.world, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.launch_count = torch.zeros(self.grid, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._hx = symm_mem.rendezvous(self.x, group)
        self._hs = symm_mem.rendezvous(self.sum, group) if result != "scatter" else None
        self._hf = symm_mem.rendezvous(self.flags, group)
        peer_form = mode == _lib.ALLREDUCE_PEER or (mode == _lib.ALLREDUCE_AUTO and self.world in (2, 4))
        for h in (self._hx, self._hs):
            if h is not None and not peer_form and not h.multicast_ptr:
                raise RuntimeError("this system gives no NVSwitch multicast mapping: use the NCCL all-reduce")
        torch.cuda.synchronize(device)
        self._hf.barrier()          # every rank's flags are zero before anybody signals

    def __call__(self, residual: torch.Tensor, weight: torch.Tensor = None, eps: float = 0.0):
        """``self.x`` holds this rank's partial output.  Returns (sum, norm): ``sum`` = residual + sum over
        ranks (all rows, or the owned rows for ``scatter``), ``norm`` its RMSNorm or None."""
        if residual.shape != self.x.shape or residual.dtype != self.x.dtype or not residual.is_contiguous():
            raise ValueError("residual must match the symmetric buffer")
        if self.norm is not None and weight is None:
            raise ValueError("the all-reduce + norm result needs the norm weight")
        hs = self._hs
        common = (
            ctypes.c_void_p(self._hx.multicast_ptr or None), ctypes.c_void_p(self._hx.buffer_ptrs_dev),
            ctypes.c_void_p(residual.data_ptr()), ctypes.c_void_p(0 if weight is None else weight.data_ptr()),
            ctypes.c_void_p((hs.multicast_ptr or None) if hs is not None else None),
            ctypes.c_void_p(hs.buffer_ptrs_dev if hs is not None else None),
            ctypes.c_void_p(self._out_ptr), ctypes.c_void_p(0 if self.norm is None else self.norm.data_ptr()),
            ctypes.c_void_p(self._hf.buffer_ptrs_dev),
            ctypes.c_void_p(self.launch_count.data_ptr()), self.rank, self.world, self.rows, self.cols, eps,
            self.mode)
        tail = (ctypes.c_void_p(self.status.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if self.schedule == "pipelined":
            check(_lib.load().ktk_exchange_rows(*common, RESULTS[self.result], *tail))
        else:
            check(_lib.load().ktk_allreduce_add_rmsnorm(*common, *tail))
        ops._launched()
        return self.sum, self.norm


class FusedAllReduceNorm(FusedExchange):
    """All-reduce + residual add + RMSNorm (the o_proj exchange)."""

    def __init__(self, group, rows: int, cols: int, dtype, device, mode: int = _lib.ALLREDUCE_AUTO,
                 schedule: str = None):
        super().__init__(group, rows, cols, dtype, device, mode=mode, result="allreduce_norm", schedule=schedule)


class RankBarrier:
    """``ktk_rank_barrier`` with its flags: a stream-ordered meeting point of the ranks (bounded wait)."""

    def __init__(self, group, device):
        import torch.distributed._symmetric_memory as symm_mem

        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.flags = symm_mem.empty(self.world, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.launch_count = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._hf = symm_mem.rendezvous(self.flags, group)
        torch.cuda.synchronize(device)
        self._hf.barrier()

    def __call__(self):
        check(_lib.load().ktk_rank_barrier(ctypes.c_void_p(self._hf.buffer_ptrs_dev),
                                           ctypes.c_void_p(self.launch_count.data_ptr()), self.rank, self.world,
                                           ctypes.c_void_p(self.status.data_ptr()),
                                           ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        ops._launched()


class SharedRows:
    """A [rows, cols] buffer on every rank whose row slices the ranks fill for one another with copy-engine
    peer copies (an all-gather without a kernel): rank r writes rows [r*rows/N, (r+1)*rows/N) everywhere."""

    def __init__(self, group, rows: int, cols: int, dtype, device):
        import torch.distributed._symmetric_memory as symm_mem

        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if rows % self.world:
            raise ValueError(f"{rows} rows do not divide over {self.world} ranks")
        self.local = symm_mem.empty(rows, cols, dtype=dtype, device=device)
        hdl = symm_mem.rendezvous(self.local, group)
        per = rows // self.world
        self.row_range = (self.rank * per, (self.rank + 1) * per)
        self.mine = self.local[self.row_range[0]:self.row_range[1]]
        # this rank's slice inside every other rank's buffer
        self.remote = [hdl.get_buffer(p, (rows, cols), dtype)[self.row_range[0]:self.row_range[1]]
                       for p in range(self.world) if p != self.rank]
        self._hdl = hdl

    def push(self):
        """Copy this rank's slice into every other rank's buffer (asynchronous, on the current stream)."""
        for dst in self.remote:
            dst.copy_(self.mine, non_blocking=True)
