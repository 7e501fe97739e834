"""N-sharded GEMM on 2, 4 and 8 GPUs: the all-gather fused into the GEMM's epilogue (stores into the peers' full C
over NVLink) against the NCCL all-gather route and the FP32 reference, one process per GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# (M, N, K, what it exercises)
CASES = [
    (512, 1024, 4096),      # CTA pairs, staged epilogue: one TMA store per destination and chunk
    (512, 1024, 1024),      # CTA pairs, register stores
    (128, 1024, 2048),      # single CTAs (the decode shape's kind)
    (128, 512, 8192),       # single CTAs with split-K: the reducing slices store to every rank
    (384, 768, 512),        # 128 x 128 tiles
]


def _agree(ok, what, rank):
    """All ranks learn whether every rank passed; they raise (or go on) together."""
    flag = torch.tensor([1 if ok else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) == 0:
        raise AssertionError(f"rank {rank}: {what}: " + ("failed here" if not ok else "failed on another rank"))


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    from datetime import timedelta
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=timedelta(seconds=60))
    try:
        import gpu_kernels_b200 as g
        torch.backends.cuda.matmul.allow_tf32 = False
        for m, n, k in CASES:
            if (n // world) % 128:
                continue                                                             # a slab owns whole scale atoms
            gen = torch.Generator(device="cuda").manual_seed(m + n + k)              # same operands on every rank
            a = torch.randn((m, k), generator=gen, device="cuda").bfloat16()
            b = (torch.randn((n, k), generator=gen, device="cuda") * 0.02).bfloat16()
            pa, sa = g.quantize(a)
            pb, sb = g.quantize(b)
            slab, slab_scales = (t.clone() for t in g.shard_b(pb, sb, world, rank))
            ref = g.dequantize(pa, sa) @ g.dequantize(pb, sb).T
            plain = g.ShardedNvfp4Gemm(pa, sa, slab, slab_scales, split_k=True)
            want = plain.run(gather=True).clone()                                # GEMM + NCCL all-gather + strided copy
            plain.validate()
            fused = g.ShardedNvfp4Gemm(pa, sa, slab, slab_scales, split_k=True, fused_gather=True)
            for call in range(3):
                for full in fused._ipc.full:
                    full.fill_(float("nan"))
                dist.barrier()                                                   # nobody clears after a peer has written
                torch.cuda.synchronize()
                got = fused.run(gather=True)
                torch.cuda.synchronize()
                _agree(not torch.isnan(got).any(), f"{m}x{n}x{k} call {call}: unwritten part of the full C", rank)
                _agree(torch.equal(got, want), f"{m}x{n}x{k} call {call}: fused gather differs from the NCCL route", rank)
                dist.barrier()
            fused.validate()
            # A rank that lags: the odd ranks keep their stream busy (a bounded spin kernel of a few
            # milliseconds) between a run and the read of its result, while the others go straight on to the
            # next run with another alpha. The lagging rank must still read the values of ITS run: the next run
            # writes the other full-C buffer, and the run after that cannot start before the barrier.
            seen = []
            for step in range(4):
                fused.set_alpha(float(step + 1))
                got = fused.run(gather=True)
                if rank % 2:
                    torch.cuda._sleep(20_000_000)
                seen.append(got.clone())
            torch.cuda.synchronize()
            for step, c in enumerate(seen):
                plain.set_alpha(float(step + 1))
                expect = plain.run(gather=True)
                _agree(torch.equal(c, expect), f"{m}x{n}x{k} step {step}: a peer that ran ahead overwrote the result", rank)
            plain.set_alpha(1.0)
            dist.barrier()
            err = (want.float() - ref).double()
            rel = float(err.norm() / ref.double().norm())
            _agree(rel <= 1e-3, f"{m}x{n}x{k}: relative Frobenius error {rel:.3e}", rank)
            with pytest.raises(ValueError):
                fused.run(gather=False)
            fused.close()
            plain.close()
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def _peer_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    from datetime import timedelta
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=timedelta(seconds=60))
    try:
        import gpu_kernels_b200 as g
        peers = g.PeerGroup(torch.device("cuda", rank), max_ints=300)
        box = g.SharedBuffer(4 * 1024, torch.device("cuda", rank))
        mine = torch.as_tensor(g.peer.DeviceView(box.own, (1024,), "<i4"), device="cuda")
        theirs = [torch.as_tensor(g.peer.DeviceView(p, (1024,), "<i4"), device="cuda") for p in box.ptrs]
        out = torch.empty((world, 300), dtype=torch.int32, device="cuda")
        results = []
        for i in range(200):                                  # no host synchronisation inside the loop
            payload = torch.arange(300, dtype=torch.int32, device="cuda") + 1000 * rank + i
            peers.all_gather_ints(payload, out)
            # a plain store into every peer's buffer, then a barrier: the peers' values must be there after it
            for r in range(world):
                theirs[r][rank * 8:(rank + 1) * 8] = i + 1
            peers.barrier()
            results.append(mine[:world * 8].clone())
            peers.barrier()                                   # nobody overwrites before everyone has read
        torch.cuda.synchronize()
        for i, seen in enumerate(results):
            assert torch.equal(seen, torch.full((world * 8,), i + 1, dtype=torch.int32, device="cuda")), (rank, i)
        # all-gather payloads, checked with synchronisation
        for i in range(20):
            n = 1 + (i * 37) % 300
            payload = torch.arange(n, dtype=torch.int32, device="cuda") + 1000 * rank + i
            gathered = torch.empty((world, n), dtype=torch.int32, device="cuda")
            peers.all_gather_ints(payload, gathered)
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(gathered[r].cpu(), torch.arange(n, dtype=torch.int32) + 1000 * r + i), (rank, i, r)
        import ctypes
        from gpu_kernels_b200 import _lib
        assert _lib.load().gpu_kernels_nvfp4_validate(None) == 0
        box.close()
        peers.close()
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_barrier_and_gather(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    mp.spawn(_peer_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_gather(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
