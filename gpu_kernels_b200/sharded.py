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

from .gemm import Nvfp4Gemm


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


class ShardedNvfp4Gemm:
    """C[:, slab] = alpha * A @ B_slab.T on this rank; `run(gather=True)` returns the full C."""

    def __init__(self, a_packed, sfa, b_slab, sfb_slab, group=None, alpha: float = 1.0, split_k: bool = False):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.plan = Nvfp4Gemm(a_packed, b_slab, sfa, sfb_slab, alpha=alpha)
        if split_k:
            # a thin slab leaves most SMs without a tile; the library offers four units per tile for such
            # shapes (only for a process that has the GPU to itself: the units wait for each other)
            try:
                self.plan.set_option("split_k", 1)
            except RuntimeError:
                pass
        self.local = torch.empty((self.plan.m, self.plan.n), dtype=torch.float16, device=a_packed.device)
        self.full = None

    def run(self, gather: bool = False) -> torch.Tensor:
        self.plan.run(self.local)
        if not gather or self.world == 1:
            return self.local
        if self.full is None:
            self.full = torch.empty((self.plan.m, self.plan.n * self.world), dtype=torch.float16,
                                    device=self.local.device)
        return gather_columns(self.local, self.group, self.full)

    def validate(self) -> None:
        self.plan.validate()

    def close(self) -> None:
        self.plan.close()
