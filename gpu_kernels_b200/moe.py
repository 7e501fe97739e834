"""Routed-MoE expert layer in NVFP4 with expert parallelism over the GPUs of one box.

Semantics follow the reference's whole-layer oracle (reference/python/moe.py:7-26): per expert
gate_up = bf16(x W1^T), act = bf16(silu(min(g, c)) * clamp(u, -c, c) * route_weight),
out = bf16(act W2^T), per token an FP32 sum over its routes, bf16 result. Here both GEMMs run on
NVFP4 operands (weights quantised once at construction, tokens and activations quantised on the
fly, one UE4M3 scale per 16 values along K), experts are split over the ranks, and token rows
travel as quantised rows (2304 B instead of 8 KiB at H=4096) through one all-to-all each way.

The call structure mirrors the reference's `CustomMoE` (benchmarks/fused_moe.py:22-191): allocate
once, call collectively on one stream per rank, inputs may change between calls, the output tensor
is overwritten by the next call. Phases as there: metadata, FC1 (+SwiGLU), FC2, reduce.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib
from .peer import DeviceView, PeerGroup, SharedBuffer
from .nvfp4 import quantize


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def exchange_splits(counts_matrix: torch.Tensor, rank: int, local_experts: int, block_rows: int = 128):
    """Row counts of the two all-to-alls from the all-gathered route counts.

    counts_matrix [world, experts] (host): routes rank r sends to global expert e. A rank's send buffer
    is ordered by global expert id, i.e. by destination rank and, inside one destination, by its local
    expert; so the dispatch sends `send[d]` consecutive rows to rank d and receives `recv[r]` rows from
    rank r, source-major. The combine runs the same exchange backwards. Also returns the pool rows this
    rank needs (each local expert padded to whole blocks of `block_rows` rows).
    """
    world = counts_matrix.shape[0]
    per_pair = counts_matrix.view(world, world, local_experts)           # [src, dst, local expert]
    send = per_pair[rank].sum(-1).tolist()
    recv = per_pair[:, rank].sum(-1).tolist()
    expert_rows = per_pair[:, rank].sum(0)
    need = int(((expert_rows + block_rows - 1) // block_rows * block_rows).sum())
    return send, recv, need


class Nvfp4MoE:
    def __init__(self, w1: torch.Tensor, w2: torch.Tensor, num_experts: int, topk: int, clamp: float = 10.0,
                 max_tokens: int = 4096, group=None, pool_rows: int | None = None, fused: bool = True,
                 block_rows: int | None = None, exchange: str = "peer", fused_dispatch: bool = True):
        """w1 [E_local, 2I, H], w2 [E_local, H, I]: this rank's experts (bf16/fp16/fp32 CUDA tensors)."""
        if not (w1.is_cuda and w2.is_cuda):
            raise ValueError("expert weights must be CUDA tensors: this package has no CPU path")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.local_experts, two_i, self.hidden = w1.shape
        self.inter = two_i // 2
        if w2.shape != (self.local_experts, self.hidden, self.inter):
            raise ValueError("w2 must be [E_local, H, I] for w1 [E_local, 2I, H]")
        if num_experts != self.local_experts * self.world:
            raise ValueError("num_experts must equal E_local * world")
        if self.hidden % 256 or self.inter % 256:
            raise ValueError("H and I must be multiples of 256")
        if self.world > 127 or max_tokens * topk >= 1 << 24:
            # a combine destination is (rank << 24) | (route + 1) in 32 bits
            raise ValueError("at most 127 ranks and fewer than 2^24 routes per rank")
        self.experts, self.topk, self.clamp, self.max_tokens = num_experts, topk, float(clamp), max_tokens
        self.device = w1.device
        lib = _lib.load()
        self.payload = lib.gpu_kernels_nvfp4_moe_payload_bytes(self.hidden)
        # weights, quantised once along K (H for W1, I for W2); the experts are stacked along the rows.
        # For the fused FC1 epilogue W1's rows are interleaved 16 gate rows / 16 up rows, so that one lane's
        # accumulator chunk holds whole (gate, up) block pairs.
        self.fused = fused
        # exchange between ranks: "peer" = rows are stored straight into the other ranks' buffers over NVLink
        # (buffers shared through CUDA IPC, no library all-to-all, no host synchronisation); "nccl" = pack,
        # all_to_all_single, unpack (needs the split sizes on the host every call)
        if exchange not in ("peer", "nccl"):
            raise ValueError("exchange must be 'peer' or 'nccl'")
        self.exchange = exchange if self.world > 1 else "local"
        self.phase_events = None        # set to [] to record (name, cuda event) pairs during forward()
        if fused:
            w1 = (w1.reshape(self.local_experts, 2, self.inter // 16, 16, self.hidden)
                  .permute(0, 2, 1, 3, 4).reshape(self.local_experts, two_i, self.hidden))
        self.w1q, self.w1s = quantize(w1.reshape(self.local_experts * two_i, self.hidden))
        self.w2q, self.w2s = quantize(w2.reshape(self.local_experts * self.hidden, self.inter))
        # pool: worst case every route of every rank lands here, each expert padded to 128 rows
        # block_rows: rows per pool block, 128 (single-CTA tiles) or 256 (CTA pairs); None = per call, 256 once
        # an expert sees about 160 rows or more
        self.block_rows = block_rows
        # fused_dispatch: tokens are quantised inside the dispatch kernel (one CTA per token, row kept in shared
        # memory, stored straight to the experts' ranks or into the pool) instead of by the stand-alone quantiser
        # followed by a pack kernel. Same bits. Not for the all-to-all route, which packs a send buffer.
        self.fused_dispatch = fused_dispatch
        worst = self.world * max_tokens * topk + self.local_experts * 255
        self.pool_rows = pool_rows if pool_rows is not None else -(-worst // 256) * 256
        if self.pool_rows % 256:
            raise ValueError("pool_rows must be a multiple of 256")
        d, u8, i32 = self.device, torch.uint8, torch.int32
        routes = max_tokens * topk
        self.t_pad = -(-max_tokens // 128) * 128
        self.counts = torch.zeros(num_experts, dtype=i32, device=d)
        self.counts_matrix = torch.zeros((self.world, num_experts), dtype=i32, device=d)
        self.send_offset = torch.zeros(num_experts + 1, dtype=i32, device=d)
        self.seg_src = torch.zeros(self.world * self.local_experts + 1, dtype=i32, device=d)
        self.seg_pool = torch.zeros(self.world * self.local_experts, dtype=i32, device=d)
        self.block_expert = torch.zeros(self.pool_rows // 128, dtype=i32, device=d)        # sized for the smaller block
        self.block_valid = torch.zeros(self.pool_rows // 128, dtype=i32, device=d)         # real rows per block (the rest is padding)
        self.num_blocks = torch.zeros(1, dtype=i32, device=d)
        self.totals = torch.zeros(4, dtype=i32, device=d)
        self.cursor = torch.zeros(num_experts, dtype=i32, device=d)
        self.send_pos = torch.zeros(routes, dtype=i32, device=d)
        recv_cap = self.world * routes
        self.recv_cap = recv_cap
        # Buffers only some routes touch (the all-to-all route's send / receive / return rows, the unfused
        # routes' intermediates, the stand-alone quantiser's padded input) are created at first use: the
        # default route of an expert-parallel layer at 4096 tokens would otherwise hold 1.2 GB it never reads.
        bf16 = torch.bfloat16
        self._lazy_specs = {
            "x_pad": ((self.t_pad, self.hidden), bf16, True),
            "send_rows": ((routes, self.payload), u8, False),
            "recv_rows": ((recv_cap, self.payload), u8, False),
            "gate_up": ((self.pool_rows, two_i), bf16, False),
            "out_pool": ((self.pool_rows, self.hidden), bf16, False),
            "ret_send": ((recv_cap, self.hidden), bf16, False),
            "ret_recv": ((routes, self.hidden), bf16, False),
        }
        self._peer = None
        # peer exchange with the fused dispatch: packed rows go straight into the owners' pools, so the pool
        # itself is what the other ranks map, plus a side buffer for each row's scale bytes, weight and route
        self.to_pool = self.exchange == "peer" and fused_dispatch
        if self.exchange == "peer":
            self._setup_peer_buffers(routes, recv_cap)
        if not self.to_pool:
            self.pool_packed = torch.zeros((self.pool_rows, self.hidden // 2), dtype=u8, device=d)
        self.pool_scales = torch.zeros(self.pool_rows * self.hidden // 16, dtype=u8, device=d)
        self.pool_weight = torch.zeros(self.pool_rows, dtype=torch.float32, device=d)
        self.pool_of_recv = torch.zeros(recv_cap, dtype=i32, device=d)
        self.act_packed = torch.empty((self.pool_rows, self.inter // 2), dtype=u8, device=d)
        self.act_scales = torch.empty(self.pool_rows * self.inter // 16, dtype=u8, device=d)
        self.y = torch.empty((max_tokens, self.hidden), dtype=torch.bfloat16, device=d)
        self._plans = {}
        with torch.cuda.device(d):
            for rows in (128, 256):
                fc1, fc2 = ctypes.c_void_p(), ctypes.c_void_p()
                _lib.check(lib.gpu_kernels_nvfp4_grouped_plan_create(
                    ctypes.byref(fc1), self.pool_rows, two_i, self.hidden, self.local_experts, rows,
                    self.pool_packed.data_ptr(), self.w1q.data_ptr(), self.pool_scales.data_ptr(), self.w1s.data_ptr(),
                    self.block_expert.data_ptr(), self.num_blocks.data_ptr()))
                _lib.check(lib.gpu_kernels_nvfp4_grouped_plan_create(
                    ctypes.byref(fc2), self.pool_rows, self.hidden, self.inter, self.local_experts, rows,
                    self.act_packed.data_ptr(), self.w2q.data_ptr(), self.act_scales.data_ptr(), self.w2s.data_ptr(),
                    self.block_expert.data_ptr(), self.num_blocks.data_ptr()))
                # the plain and SwiGLU routes write only the real rows of their output pools (nobody reads the rest)
                _lib.check(lib.gpu_kernels_nvfp4_grouped_set_valid_rows(fc1, self.block_valid.data_ptr()))
                _lib.check(lib.gpu_kernels_nvfp4_grouped_set_valid_rows(fc2, self.block_valid.data_ptr()))
                self._plans[rows] = (fc1, fc2)

    def __getattr__(self, name):
        # only reached for attributes that do not exist yet: the lazily created buffers
        specs = self.__dict__.get("_lazy_specs")
        if specs and name in specs:
            shape, dtype, zero = specs[name]
            make = torch.zeros if zero else torch.empty
            tensor = make(shape, dtype=dtype, device=self.__dict__["device"])
            self.__dict__[name] = tensor
            return tensor
        raise AttributeError(name)

    def _setup_peer_buffers(self, routes, recv_cap):
        """Receive and result-slot buffers that every rank of the group can write (CUDA IPC), and the barrier."""
        d = self.device
        if self.to_pool:
            pool = SharedBuffer(self.pool_rows * (self.hidden // 2), d, self.group)
            side = SharedBuffer(self.pool_rows * (self.hidden // 16 + 16), d, self.group)
            self.pool_packed = torch.as_tensor(DeviceView(pool.own, (self.pool_rows, self.hidden // 2), "|u1"), device=d)
            recv = None
        else:
            recv = SharedBuffer(recv_cap * self.payload, d, self.group)
            pool = side = None
        slots = SharedBuffer(routes * self.hidden * 2, d, self.group)
        self._peers = PeerGroup(d, self.group, max_ints=self.experts)
        self._peer = {"recv": recv, "slots": slots, "pool": pool, "side": side}
        self.recv_ptr = recv.own if recv is not None else None
        self.slots_ptr = slots.own
        self.slot_table = slots.device_table
        self.peer_offset = torch.zeros(self.experts, dtype=torch.int32, device=d)
        self.peer_error = torch.zeros(1, dtype=torch.int32, device=d)
        self.identity = torch.arange(routes, dtype=torch.int32, device=d)
        self.pool_dst = torch.zeros(self.pool_rows, dtype=torch.int32, device=d)

    def _barrier(self):
        # one small kernel per rank over peer memory: it completes on a rank only after every rank's earlier
        # work on its stream (the peer stores) has finished, and nothing on the host waits for it
        self._peers.barrier()

    def check(self) -> None:
        """Synchronises and raises if a peer store was out of bounds or the pool overflowed in the last calls."""
        torch.cuda.synchronize(self.device)
        if self._peer is not None and int(self.peer_error.item()):
            raise RuntimeError(f"expert exchange: a peer store was outside the agreed capacity (code {int(self.peer_error.item())})")
        if int(self.totals[2].item()):
            raise RuntimeError("expert pool overflow")
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_validate(None))

    def _mark(self, name):
        if self.phase_events is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.phase_events.append((name, ev))

    def phase_times_us(self):
        """Device time between the marks of the last forward() (needs phase_events = [] before the call)."""
        torch.cuda.synchronize()
        ev = self.phase_events or []
        return {ev[i + 1][0]: 1000.0 * ev[i][1].elapsed_time(ev[i + 1][1]) for i in range(len(ev) - 1)}

    # ---- phases ----------------------------------------------------------------------------------
    def _metadata(self, ids, tokens, block_rows):
        lib, s = _lib.load(), _stream()
        routes = tokens * self.topk
        if self.world == 1 and routes <= 4096:
            # one launch: histogram of the routes (by the plan's single CTA: for small batches), plan, arrival
            # counters cleared
            _lib.check(lib.gpu_kernels_nvfp4_moe_route_plan(
                ids.data_ptr(), routes, self.counts_matrix.data_ptr(), self.experts, self.pool_rows, block_rows,
                self.send_offset.data_ptr(), self.seg_src.data_ptr(), self.seg_pool.data_ptr(),
                self.block_expert.data_ptr(), self.num_blocks.data_ptr(), self.totals.data_ptr(),
                self.cursor.data_ptr(), self.block_valid.data_ptr(), s))
        else:
            if self._peer is not None and routes <= 4096:
                # small batch: histogram, peer stores of the counts and the barrier in one kernel
                st = self._peers.state
                _lib.check(lib.gpu_kernels_nvfp4_moe_count_exchange(
                    ids.data_ptr(), routes, self.experts, st.own, st.device_table.data_ptr(), self.world, self.rank,
                    self._peers.max_ints, self.counts_matrix.data_ptr(), s))
            else:
                self.counts.zero_()
                _lib.check(lib.gpu_kernels_nvfp4_moe_route_count(ids.data_ptr(), routes, self.experts, self.counts.data_ptr(), s))
                if self._peer is not None:
                    self._peers.all_gather_ints(self.counts, self.counts_matrix)      # peer stores + barrier, one kernel
                elif self.world > 1:
                    dist.all_gather_into_tensor(self.counts_matrix.view(-1), self.counts, group=self.group)
                else:
                    self.counts_matrix.copy_(self.counts.view(1, -1))
            _lib.check(lib.gpu_kernels_nvfp4_moe_plan(
                self.counts_matrix.data_ptr(), self.world, self.rank, self.experts, self.pool_rows, block_rows,
                self.send_offset.data_ptr(), self.seg_src.data_ptr(), self.seg_pool.data_ptr(),
                self.block_expert.data_ptr(), self.num_blocks.data_ptr(), self.totals.data_ptr(),
                self.peer_offset.data_ptr() if self._peer is not None else None, 1 if self.to_pool else 0,
                self.cursor.data_ptr(), self.block_valid.data_ptr(), s))
        # padding rows of the live blocks must contribute nothing: clear their scale bytes, weights and codes
        _lib.check(lib.gpu_kernels_nvfp4_moe_clear_live(
            self.num_blocks.data_ptr(), block_rows, self.pool_rows, self.hidden, self.pool_scales.data_ptr(),
            self.pool_weight.data_ptr(), self.pool_dst.data_ptr() if self._peer is not None else None, s))
        if self._peer is not None and self.pool_rows >= self.world * self.max_tokens * self.topk + self.local_experts * (block_rows - 1):
            # peer exchange with a worst-case pool: the host needs nothing from the counts
            return None, None
        if self.world == 1 and self.pool_rows >= routes + self.local_experts * (block_rows - 1):
            # one rank, pool sized for the worst case: nothing to exchange and nothing can overflow, so the
            # host never has to look at the counts and the whole forward stays asynchronous
            return [routes], [routes]
        # the split sizes of the all-to-all have to be host integers: one small D2H copy per call
        send_splits, recv_splits, need = exchange_splits(self.counts_matrix.cpu(), self.rank, self.local_experts, block_rows)
        if need > self.pool_rows:
            raise RuntimeError(f"expert pool overflow: {need} rows needed, {self.pool_rows} allocated")
        return send_splits, recv_splits

    def forward(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """x [T, H] bf16, ids [T, topk] int64 global expert ids, weights [T, topk] f32 -> y [T, H] bf16.

        A route whose id lies outside [0, num_experts) (a router's "dropped" mark such as -1) is dropped: no row
        is dispatched for it and it adds nothing to its token's sum, on every exchange route."""
        tokens = x.shape[0]
        if tokens > self.max_tokens or x.shape[1] != self.hidden or ids.shape != (tokens, self.topk):
            raise ValueError("shape mismatch with the layer this object was built for")
        lib = _lib.load()
        ids = ids.contiguous().to(torch.int64)
        weights = weights.contiguous().to(torch.float32)
        with torch.cuda.device(self.device):
            s = _stream()
            fused_dispatch = self.fused_dispatch and (self.world == 1 or self._peer is not None)
            self._mark("start")
            if not fused_dispatch:
                # quantise the tokens once; rows are padded to whole 128-row scale atoms
                self.x_pad[:tokens].copy_(x)
                xq, xs = quantize(self.x_pad)
                self._mark("quantise tokens")
            # rows an expert of this rank sees on average decide the block size (and with it single CTAs or pairs)
            block_rows = self.block_rows or (256 if tokens * self.topk * self.world >= 160 * self.experts else 128)
            fc1, fc2 = self._plans[block_rows]
            send_splits, recv_splits = self._metadata(ids, tokens, block_rows)
            self._mark("metadata (counts, all-gather, plan, host split sizes)")
            if fused_dispatch and self.world > 1 and send_splits is not None:
                # a pool below the worst case sends this call through the all-to-all route, which packs a send buffer
                fused_dispatch = False
                self.x_pad[:tokens].copy_(x)
                xq, xs = quantize(self.x_pad)
            total_recv = sum(recv_splits) if recv_splits is not None else 0
            if fused_dispatch and (self.world == 1 or send_splits is None):
                x = x.to(torch.bfloat16).contiguous()             # as the stand-alone route's padded copy does
                peer = self.world > 1
                if peer and self.to_pool:
                    targets, side, capacity = self._peer["pool"].table, self._peer["side"].table, self.pool_rows
                elif peer:
                    targets, side, capacity = self._peer["recv"].table, None, self.recv_cap
                else:
                    targets, side, capacity = None, None, 0
                _lib.check(lib.gpu_kernels_nvfp4_moe_quantise_route(
                    x.data_ptr(), ids.data_ptr(), weights.data_ptr(), tokens, self.topk, self.hidden, self.experts,
                    (self.peer_offset if peer else self.seg_pool).data_ptr(), self.cursor.data_ptr(),
                    targets, side, self.world if peer else 0, self.local_experts,
                    capacity, self.peer_error.data_ptr() if peer else None,
                    None if peer else self.pool_packed.data_ptr(), None if peer else self.pool_scales.data_ptr(),
                    None if peer else self.pool_weight.data_ptr(), None if peer else self.send_pos.data_ptr(), s))
                if peer:
                    self._mark("quantise + pack into the peers' receive buffers")
                    self._barrier()
                    self._mark("barrier")
                    if self.to_pool:
                        # the packed rows are already in place: only scale atoms, weights and destinations are left
                        _lib.check(lib.gpu_kernels_nvfp4_moe_unpack_meta(
                            self._peer["side"].own, self.recv_cap, self.totals.data_ptr(), self.world, self.local_experts,
                            self.hidden, self.seg_src.data_ptr(), self.seg_pool.data_ptr(), self.pool_scales.data_ptr(),
                            self.pool_weight.data_ptr(), self.pool_dst.data_ptr(), s))
                    else:
                        _lib.check(lib.gpu_kernels_nvfp4_moe_unpack(
                            self.recv_ptr, self.recv_cap, self.totals.data_ptr(), self.world, self.local_experts,
                            self.hidden, self.seg_src.data_ptr(), self.seg_pool.data_ptr(), self.pool_packed.data_ptr(),
                            self.pool_scales.data_ptr(), self.pool_weight.data_ptr(), self.pool_of_recv.data_ptr(),
                            self.pool_dst.data_ptr(), s))
            elif self.world > 1 and send_splits is None:
                _lib.check(lib.gpu_kernels_nvfp4_moe_pack_peer(
                    xq.data_ptr(), xs.data_ptr(), ids.data_ptr(), weights.data_ptr(), tokens, self.topk, self.hidden,
                    self.world, self.local_experts, self.peer_offset.data_ptr(), self.cursor.data_ptr(),
                    self._peer["recv"].table, self.recv_cap, self.peer_error.data_ptr(), s))
                self._mark("pack into the peers' receive buffers")
                self._barrier()
                self._mark("barrier")
                _lib.check(lib.gpu_kernels_nvfp4_moe_unpack(
                    self.recv_ptr, self.recv_cap, self.totals.data_ptr(), self.world, self.local_experts,
                    self.hidden, self.seg_src.data_ptr(), self.seg_pool.data_ptr(), self.pool_packed.data_ptr(),
                    self.pool_scales.data_ptr(), self.pool_weight.data_ptr(), self.pool_of_recv.data_ptr(),
                    self.pool_dst.data_ptr(), s))
            elif self.world == 1:
                # nothing to exchange: rows go straight into the expert-major pool
                _lib.check(lib.gpu_kernels_nvfp4_moe_pack_to_pool(
                    xq.data_ptr(), xs.data_ptr(), ids.data_ptr(), weights.data_ptr(), tokens, self.topk, self.hidden,
                    self.experts, self.seg_pool.data_ptr(), self.cursor.data_ptr(), self.pool_packed.data_ptr(),
                    self.pool_scales.data_ptr(), self.pool_weight.data_ptr(), self.send_pos.data_ptr(), s))
            else:
                _lib.check(lib.gpu_kernels_nvfp4_moe_pack(
                    xq.data_ptr(), xs.data_ptr(), ids.data_ptr(), weights.data_ptr(), tokens, self.topk, self.hidden,
                    self.experts, self.send_offset.data_ptr(), self.cursor.data_ptr(), self.send_rows.data_ptr(),
                    self.send_pos.data_ptr(), s))
                self._mark("pack")
                dist.all_to_all_single(self.recv_rows[:total_recv], self.send_rows[:tokens * self.topk],
                                       recv_splits, send_splits, group=self.group)
                self._mark("dispatch all-to-all")
                _lib.check(lib.gpu_kernels_nvfp4_moe_unpack(
                    self.recv_rows.data_ptr(), self.recv_cap, self.totals.data_ptr(), self.world, self.local_experts,
                    self.hidden, self.seg_src.data_ptr(), self.seg_pool.data_ptr(), self.pool_packed.data_ptr(),
                    self.pool_scales.data_ptr(), self.pool_weight.data_ptr(), self.pool_of_recv.data_ptr(), None, s))
            self._mark("pool filled")
            if self.fused:
                _lib.check(lib.gpu_kernels_nvfp4_grouped_run_swiglu(
                    fc1, self.pool_weight.data_ptr(), self.clamp, self.act_packed.data_ptr(),
                    self.act_scales.data_ptr(), s))
            else:
                _lib.check(lib.gpu_kernels_nvfp4_grouped_run(fc1, self.gate_up.data_ptr(), 1, s))
                _lib.check(lib.gpu_kernels_nvfp4_moe_swiglu_quant(
                    self.gate_up.data_ptr(), self.pool_weight.data_ptr(), self.num_blocks.data_ptr(), block_rows, self.pool_rows,
                    self.inter, self.clamp, self.act_packed.data_ptr(), self.act_scales.data_ptr(), s))
            self._mark("FC1 + SwiGLU + quantise")
            peer = self.world > 1 and send_splits is None
            if peer:
                # FC2 fused with the combine: every output row leaves the epilogue for its token's rank
                _lib.check(lib.gpu_kernels_nvfp4_grouped_run_scatter(
                    fc2, self.pool_dst.data_ptr(), self.slot_table.data_ptr(), self.slots_ptr, self.world,
                    self.max_tokens * self.topk, 1, s))
            else:
                _lib.check(lib.gpu_kernels_nvfp4_grouped_run(fc2, self.out_pool.data_ptr(), 1, s))
            self._mark("FC2")
            if peer:
                self._mark("expert outputs into the sources' slot buffers")
                self._barrier()
                self._mark("barrier")
                _lib.check(lib.gpu_kernels_nvfp4_moe_reduce(
                    self.slots_ptr, self.identity.data_ptr(), tokens, self.topk, self.hidden, self.y.data_ptr(),
                    ids.data_ptr(), self.experts, s))
            elif self.world == 1:
                # send_pos holds pool rows: the reduce reads the second GEMM's output in place
                _lib.check(lib.gpu_kernels_nvfp4_moe_reduce(
                    self.out_pool.data_ptr(), self.send_pos.data_ptr(), tokens, self.topk, self.hidden,
                    self.y.data_ptr(), ids.data_ptr(), self.experts, s))
            else:
                _lib.check(lib.gpu_kernels_nvfp4_moe_return_rows(
                    self.out_pool.data_ptr(), self.pool_of_recv.data_ptr(), self.totals.data_ptr(), self.recv_cap,
                    self.hidden, self.ret_send.data_ptr(), s))
                self._mark("return_rows")
                dist.all_to_all_single(self.ret_recv[:tokens * self.topk].view(torch.uint8),
                                       self.ret_send[:total_recv].view(torch.uint8),
                                       send_splits, recv_splits, group=self.group)
                self._mark("combine all-to-all")
                _lib.check(lib.gpu_kernels_nvfp4_moe_reduce(
                    self.ret_recv.data_ptr(), self.send_pos.data_ptr(), tokens, self.topk, self.hidden,
                    self.y.data_ptr(), ids.data_ptr(), self.experts, s))
            self._mark("reduce")
        return self.y[:tokens]

    __call__ = forward

    def capture(self, tokens: int):
        """Records forward() for `tokens` tokens as one CUDA graph (kernels, collectives and peer stores).

        Returns (x, ids, weights, y, graph): write the inputs into the first three (device tensors of the shapes
        forward() takes), call graph.replay(), read y (a view of the layer's output buffer). Possible where
        forward() needs nothing from the host: one rank, or the peer exchange, with the pool at its worst-case
        size (the default). Every rank of the group captures (token counts may differ) and then replays the same
        number of times, as with any collective."""
        if tokens < 1 or tokens > self.max_tokens:
            raise ValueError("tokens outside 1..max_tokens")
        if self.world > 1 and self._peer is None:
            raise RuntimeError("capture needs exchange='peer': the all-to-all path reads its split sizes on the host")
        worst = self.world * self.max_tokens * self.topk + self.local_experts * 255
        if self.pool_rows < worst:
            raise RuntimeError(f"capture needs a worst-case pool ({worst} rows): a smaller one is checked on the host")
        if self.phase_events is not None:
            raise RuntimeError("phase timing marks cannot be captured")
        d = self.device
        x = torch.zeros((tokens, self.hidden), dtype=torch.bfloat16, device=d)
        ids = torch.zeros((tokens, self.topk), dtype=torch.int64, device=d)
        weights = torch.zeros((tokens, self.topk), dtype=torch.float32, device=d)
        with torch.cuda.device(d):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):                       # first calls: library load, communicator, plans
                for _ in range(2):
                    self.forward(x, ids, weights)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize(d)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                y = self.forward(x, ids, weights)
        return x, ids, weights, y, graph

    def close(self) -> None:
        lib = _lib.load()
        if self._peer is not None:
            if self.to_pool:
                del self.pool_packed                            # a view of the shared pool, freed below
            self._peers.close()
            for name in ("slots", "recv", "pool", "side"):
                if self._peer[name] is not None:
                    self._peer[name].close()
            self._peer = None
        for pair in getattr(self, "_plans", {}).values():
            for plan in pair:
                if plan:
                    lib.gpu_kernels_nvfp4_grouped_plan_destroy(plan)
        self._plans = {}

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def route(logits: torch.Tensor, topk: int):
    """softmax over router logits, top-k, weights renormalised to sum 1 (the benchmark's routing)."""
    prob = torch.softmax(logits.float(), dim=-1)
    weights, ids = prob.topk(topk, dim=-1)
    return ids, weights / weights.sum(-1, keepdim=True)
