"""N-column sharding of the NVFP4 GEMM across the GPUs of one box.

Rank g of G holds rows [g*N/G, (g+1)*N/G) of B (packed values and scale bytes)
and the whole of A; it computes the column slab C[:, g*N/G:(g+1)*N/G] with no
exchange. `gather_columns` is the optional NCCL all-gather that rebuilds the full
C on every rank when the caller asks for it. The reference's GEMM is single-GPU
(kernels/gemm/matmul/sm100.cu:728-731); this layer is new and keeps its operand
layout, so a slab of B is just a row range of the reference's tensors: slabs of
a multiple of 128 rows own whole scale atoms.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from .gemm import Nvfp4Gemm
from .peer import DeviceView, PeerGroup, SharedBuffer


def slab_rows(n: int, world: int, rank: int) -> tuple[int, int]:
    """Row range [lo, hi) of B that `rank` owns. N/world must be a multiple of 128."""
    if n % world:
        raise ValueError(f"N={n} does not divide over {world} ranks")
    per = n // world
    if per % 128:
        raise ValueError(f"N/world={per} must be a multiple of 128 (whole scale atoms per slab)")
    return rank * per, (rank + 1) * per


def shard_b(b_packed: torch.Tensor, sfb: torch.Tensor, world: int, rank: int):
    """Slice a full B [N, K/2] and its VEC16 scale bytes down to this rank's slab (views, no copy)."""
    n, half_k = b_packed.shape
    lo, hi = slab_rows(n, world, rank)
    per_row = half_k // 8                      # scale bytes per row = K/16
    return b_packed[lo:hi], sfb[lo * per_row:hi * per_row]


def gather_columns(local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather column slabs [M, N/G] into the full row-major [M, N] on every rank.

    One all_gather_into_tensor (NCCL on GPUs, gloo on CPU tensors) into a
    [G, M, N/G] staging buffer, then one strided copy into row-major order.
    """
    world = dist.get_world_size(group)
    m, per = local.shape
    stage = torch.empty((world * m, per), dtype=local.dtype, device=local.device)
    # moved as raw bytes: every backend (NCCL, gloo) handles uint8
    dist.all_gather_into_tensor(stage.view(torch.uint8), local.contiguous().view(torch.uint8), group=group)
    if out is None:
        out = torch.empty((m, world * per), dtype=local.dtype, device=local.device)
    out.view(m, world, per).copy_(stage.view(world, m, per).permute(1, 0, 2))
    return out


class GatheredOutput:
    """Full [M, N_total] C buffers (FP16, or BF16 with dtype=torch.bfloat16) on every rank of the group, each
    mapped into all the others (CUDA IPC).

    `attach(plan, col0, index)` makes a plan's epilogue write its column slab into buffer `index` of every
    rank (this rank's own and, over NVLink, the peers'); `barrier()` is the stream-ordered point after which
    every rank's stores have landed. There are two buffers, used in turn (`turn()` hands out the index of the
    next run): a rank that is one step ahead then writes the other buffer, not the one a slower rank is still
    reading, and it cannot get two steps ahead because the barrier in between needs the slower rank. So one
    barrier per run is enough, as long as every rank reads a result, on the stream it runs on, before it starts
    its next run. All ranks must sit on one NVLink node. Collective: construct and close on every rank.
    """

    def __init__(self, m: int, n_total: int, device, group=None, dtype=torch.float16, buffers: int = 2):
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("the full C is float16 or bfloat16")
        self.m, self.n_total, self.dtype = m, n_total, dtype
        self.buffers = [SharedBuffer(m * n_total * 2, device, group) for _ in range(buffers)]
        self.peers = PeerGroup(device, group, max_ints=0)
        self.device = self.buffers[0].device
        self.world = self.buffers[0].world
        self.full = [torch.as_tensor(DeviceView(b.own, (m, n_total), "<i2"), device=self.device).view(dtype)
                     for b in self.buffers]
        self._turn = 0

    def attach(self, plan: Nvfp4Gemm, col0: int, index: int = 0) -> None:
        if plan.m != self.m:
            raise ValueError("plan and output disagree on M")
        if plan.out_dtype != self.dtype:
            raise ValueError("plan and output disagree on the element type")
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_plan_set_gather(plan._plan, self.buffers[index].table, self.world,
                                                                     col0, self.n_total))

    def turn(self) -> int:
        """Index of the buffer the next run writes (every rank calls this once per run, in step)."""
        index = self._turn % len(self.buffers)
        self._turn += 1
        return index

    def barrier(self) -> None:
        self.peers.barrier()

    def close(self) -> None:
        if self.full is None:
            return
        self.full = None
        self.peers.close()
        for b in self.buffers:
            b.close()


class ShardedNvfp4Gemm:
    """C[:, slab] = alpha * A @ B_slab.T on this rank; `run(gather=True)` returns the full C on every rank.

    fused_gather=True (all ranks on one NVLink node): the full C of every rank lives in buffers the other
    ranks map through CUDA IPC, and the GEMM's epilogue writes this rank's slab into all of them while the
    tiles are computed; run(gather=True) is then that one kernel plus a barrier kernel over peer memory
    (stream-ordered, nothing for the host to wait on). Two full-C buffers are written in turn, so a rank that
    runs ahead never overwrites the result a slower rank is still reading: the tensor a run returns stays
    valid until this rank's second run after it; consume it on the same stream before calling run() again.
    `gathered` lets several objects (operand sets of one shape) share one pair of buffers and one turn counter.
    Otherwise run(gather=True) is the GEMM, an NCCL all-gather and a strided copy into one reused tensor.
    """

    def __init__(self, a_packed, sfa, b_slab, sfb_slab, group=None, alpha: float = 1.0, split_k: bool = False,
                 fused_gather: bool = False, gathered: GatheredOutput | None = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._operands = (a_packed, b_slab, sfa, sfb_slab)
        self._alpha, self._split_k = alpha, split_k
        self.plan = self._make_plan()
        self.local = torch.empty((self.plan.m, self.plan.n), dtype=torch.float16, device=a_packed.device)
        self.full = None
        self._ipc, self._owns_ipc, self._plans = None, False, None
        if (fused_gather or gathered is not None) and self.world > 1:
            self._ipc = gathered
            if self._ipc is None:
                self._ipc = GatheredOutput(self.plan.m, self.plan.n * self.world, self.local.device, self.group)
                self._owns_ipc = True
            # one plan per buffer: the destination table is part of a plan
            self._plans = [self.plan] + [self._make_plan() for _ in range(len(self._ipc.buffers) - 1)]
            for index, plan in enumerate(self._plans):
                self._ipc.attach(plan, self.rank * self.plan.n, index)

    def _make_plan(self) -> Nvfp4Gemm:
        a, b, sfa, sfb = self._operands
        plan = Nvfp4Gemm(a, b, sfa, sfb, alpha=self._alpha)
        if self._split_k:
            # a thin slab leaves most SMs without a tile; the library offers four units per tile for such
            # shapes (only for a process that has the GPU to itself: the units wait for each other)
            try:
                plan.set_option("split_k", 1)
            except RuntimeError:
                pass
        return plan

    def run(self, gather: bool = False) -> torch.Tensor:
        if self._ipc is not None:
            if not gather:
                raise ValueError("this object was built with fused_gather=True: every run writes the full C")
            index = self._ipc.turn()
            self._plans[index].run(self.local)          # the slab goes to every rank's full C; `local` stays untouched
            self._ipc.barrier()                         # all ranks' stores have landed once this completes
            self.full = self._ipc.full[index]
            return self.full
        self.plan.run(self.local)
        if not gather or self.world == 1:
            return self.local
        if self.full is None:
            self.full = torch.empty((self.plan.m, self.plan.n * self.world), dtype=torch.float16,
                                    device=self.local.device)
        return gather_columns(self.local, self.group, self.full)

    def set_alpha(self, alpha: float) -> None:
        for plan in self._plans or [self.plan]:
            plan.set_alpha(alpha)

    def validate(self) -> None:
        for plan in self._plans or [self.plan]:
            plan.validate()

    def close(self) -> None:
        if self._ipc is not None:
            self.full = None
            if self._owns_ipc:
                self._ipc.close()
            self._ipc = None
        for plan in self._plans or [self.plan]:
            plan.close()
        self._plans = None
