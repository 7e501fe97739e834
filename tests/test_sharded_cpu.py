"""N-sharding host logic on two gloo ranks (CPU). The local GEMM of each rank is
stood in for by the oracle, which is allowed here because this file is a test."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nvfp4_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gpu_kernels_b200.sharded import gather_columns, shard_b
        rng = np.random.default_rng(3)
        m, n, k = 128, 512, 256
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        pa, sa = O.quantize(a)
        pb, sb = O.quantize(b)
        slab_p, slab_s = shard_b(torch.from_numpy(pb), torch.from_numpy(sb), world, rank)
        # a slab of B is self-contained: quantising the slab's rows alone gives the same bytes
        lo, hi = rank * n // world, (rank + 1) * n // world
        p2, s2 = O.quantize(b[lo:hi])
        assert np.array_equal(slab_p.numpy(), p2) and np.array_equal(slab_s.numpy(), s2)
        local = torch.from_numpy(O.gemm(pa, sa, slab_p.numpy(), slab_s.numpy()))
        full = gather_columns(local)
        want = O.gemm(pa, sa, pb, sb)
        assert np.array_equal(full.numpy().view(np.uint16)[:, lo:hi], want.view(np.uint16)[:, lo:hi])
        assert np.abs(full.numpy().astype(np.float32) - want.astype(np.float32)).max() <= 2 ** -8 * np.abs(want).max()
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_slab_rows_rules():
    from gpu_kernels_b200.sharded import slab_rows
    assert slab_rows(28672, 8, 3) == (3 * 3584, 4 * 3584)
    with pytest.raises(ValueError):
        slab_rows(8192, 3, 0)
    with pytest.raises(ValueError):
        slab_rows(512, 8, 0)
