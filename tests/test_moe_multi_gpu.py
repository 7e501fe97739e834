"""Expert parallelism over 2, 4 and 8 GPUs (stores into the peers' memory, and NCCL all-to-all each way) against
the CPU oracle, one process per GPU. As in the reference's multi-GPU check (benchmarks/moe_pipeline.py:71-82,
130-156): every rank count, a rerun with changed inputs through the same object, and a verdict the ranks share
through an all-reduce, so that a failure on one rank ends all of them together instead of leaving the others in
a collective. Skipped where fewer GPUs are visible."""
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
        from oracle import moe_oracle as MO
        hidden, inter, experts, topk = 512, 256, 16, 2
        local = experts // world
        gen = torch.Generator(device="cuda").manual_seed(100)                # same weights on every rank
        w1 = (torch.randn((experts, 2 * inter, hidden), generator=gen, device="cuda") * 0.02).bfloat16()
        w2 = (torch.randn((experts, hidden, inter), generator=gen, device="cuda") * 0.02).bfloat16()
        outputs = {}
        for exchange, fused_dispatch in (("peer", True), ("peer", False), ("nccl", False)):
            layer = g.Nvfp4MoE(w1[rank * local:(rank + 1) * local], w2[rank * local:(rank + 1) * local], experts, topk,
                               max_tokens=128, exchange=exchange, fused_dispatch=fused_dispatch)
            for call, tokens in enumerate((50 + 11 * rank, 7, 128)):               # ragged token counts (at most 127); the last call uses 256-row blocks
                gen_r = torch.Generator(device="cuda").manual_seed(1000 * call + rank)
                x = torch.randn((tokens, hidden), generator=gen_r, device="cuda").bfloat16()
                ids, wts = g.route(torch.randn((tokens, experts), generator=gen_r, device="cuda"), topk)
                layer.block_rows = 256 if call == 2 else None
                try:                                                               # an exception here is a verdict too
                    y = layer(x, ids, wts)
                    torch.cuda.synchronize()
                    ref = MO.moe_forward_nvfp4(x.float().cpu().numpy(), ids.cpu().numpy(), wts.cpu().numpy(),
                                               w1.float().cpu().numpy(), w2.float().cpu().numpy(), 10.0)
                    got = y.float().cpu().numpy()
                    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
                    ok, what = bool(not np.isnan(got).any() and rel <= 2e-2), f"rel {rel:.3e}"
                except Exception as exc:                                           # noqa: BLE001
                    got, ok, what = np.zeros((tokens, hidden), np.float32), False, f"{type(exc).__name__}: {exc}"
                _agree(ok, f"{exchange} call {call}: {what}", rank)
                # both exchanges deliver the same rows and the reduce adds them in the same order: identical bits
                _agree(np.array_equal(outputs.setdefault(call, got), got),
                       f"call {call}: {exchange} fused_dispatch={fused_dispatch} differs from the first exchange", rank)
            if exchange == "peer" and fused_dispatch:
                # the same forward, collectives and peer stores included, replayed from a CUDA graph
                gx, gids, gwts, gy, graph = layer.capture(tokens)
                for _ in range(2):
                    gx.copy_(x); gids.copy_(ids); gwts.copy_(wts)
                    graph.replay()
                    torch.cuda.synchronize()
                    _agree(np.array_equal(gy.float().cpu().numpy(), outputs[2]), "graph replay differs", rank)
                del graph
            layer.check()
            layer.close()
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
