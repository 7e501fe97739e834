"""Expert-parallel exchange protocol on two gloo ranks (CPU).

The product's host logic here is `exchange_splits` (row counts of the all-to-alls) and the ordering
contract around it: a rank's send buffer is ordered by global expert id; the receive buffer is then
source-major with each source's rows in local-expert order; the plan kernel's segment tables are
prefix sums over the same count matrix. The CUDA kernels cannot run here, so rows are stand-ins that
carry (source rank, route id, expert) and the test restates the plan's prefix sums in numpy.
"""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gpu_kernels_b200.moe import exchange_splits
        experts, topk, tokens = 8, 3, 21 + 5 * rank
        local = experts // world
        rng = np.random.default_rng(10 + rank)
        ids = np.stack([rng.choice(experts, size=topk, replace=False) for _ in range(tokens)])
        counts = torch.from_numpy(np.bincount(ids.reshape(-1), minlength=experts).astype(np.int32))
        gathered = [torch.zeros_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts)
        matrix = torch.stack(gathered)
        send, recv, need = exchange_splits(matrix, rank, local)
        assert sum(send) == tokens * topk
        # pack: rows ordered by global expert (stable inside an expert here; the kernel's order inside an
        # expert is arbitrary, which the checks below do not depend on)
        order = np.argsort(ids.reshape(-1), kind="stable")
        rows = np.stack([np.full(len(order), rank), order, ids.reshape(-1)[order]], axis=1).astype(np.int64)
        recv_rows = torch.zeros((sum(recv), 3), dtype=torch.int64)
        dist.all_to_all_single(recv_rows, torch.from_numpy(rows), recv, send)
        got = recv_rows.numpy()
        # the plan's tables, restated: segments (source r, local expert e) in source-major order
        m = matrix.numpy()
        mine = m[:, rank * local:(rank + 1) * local]                        # [source, local expert]
        seg_start = np.concatenate(([0], np.cumsum(mine.reshape(-1))))
        for r in range(world):
            for e in range(local):
                seg = got[seg_start[r * local + e]:seg_start[r * local + e + 1]]
                assert (seg[:, 0] == r).all() and (seg[:, 2] == rank * local + e).all()
        padded = (mine.sum(0) + 127) // 128 * 128
        assert need == padded.sum()
        # combine: the same exchange backwards returns every row to the rank and position it came from
        back = torch.zeros((sum(send), 3), dtype=torch.int64)
        dist.all_to_all_single(back, recv_rows, send, recv)
        assert np.array_equal(back.numpy(), rows)
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_dispatch_and_combine(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
