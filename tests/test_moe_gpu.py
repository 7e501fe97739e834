"""NVFP4 routed-MoE expert path on one GPU (expert parallelism 1) against the CPU oracle.

Integer/byte stages (routing plan, pack, unpack, reduce order) are checked exactly; the two grouped
GEMMs and the activation are floating point with bf16 rounding points, compared within the stated
tolerances against `oracle.moe_oracle.moe_forward_nvfp4` (FP32 dequantise-then-matmul).
"""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as MO
from oracle import nvfp4_oracle as O
from helpers import to_np

pytestmark = pytest.mark.gpu

# Floating-point acceptance for the whole layer (bf16 output, two quantised GEMMs in sequence):
# relative Frobenius error and max abs error over output RMS. A 1-ulp bf16 difference in gate_up
# (FP32 summation order) can flip an E2M1 code of the re-quantised activation, which moves single
# outputs by a quantisation step times a weight, hence looser than the single-GEMM bound.
LAYER_REL_FROBENIUS = 2e-2
LAYER_MAX_ABS_OVER_RMS = 0.25


@pytest.fixture(scope="module")
def g():
    import gpu_kernels_b200
    return gpu_kernels_b200


def make_layer(seed, tokens, hidden, inter, experts, topk, skew=False):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((tokens, hidden), generator=gen, device="cuda").bfloat16()
    logits = torch.randn((tokens, experts), generator=gen, device="cuda")
    if skew:
        logits[:, 0] += 4.0                                  # most tokens pick expert 0; some experts stay empty
        logits[:, experts // 2:] -= 8.0
    w1 = (torch.randn((experts, 2 * inter, hidden), generator=gen, device="cuda") * 0.02).bfloat16()
    w2 = (torch.randn((experts, hidden, inter), generator=gen, device="cuda") * 0.02).bfloat16()
    return x, logits, w1, w2


def oracle_layer(x, ids, wts, w1, w2, clamp):
    return MO.moe_forward_nvfp4(to_np(x.float()), to_np(ids), to_np(wts), to_np(w1.float()), to_np(w2.float()), clamp)


def assert_layer_close(y, ref, what):
    y = to_np(y.float()).astype(np.float64)
    ref = ref.astype(np.float64)
    assert not np.isnan(y).any(), f"{what}: NaN in the output"
    rel = np.linalg.norm(y - ref) / max(np.linalg.norm(ref), 1e-30)
    worst = np.abs(y - ref).max() / max(np.sqrt((ref ** 2).mean()), 1e-30)
    assert rel <= LAYER_REL_FROBENIUS, f"{what}: relative Frobenius error {rel:.3e}"
    assert worst <= LAYER_MAX_ABS_OVER_RMS, f"{what}: max abs error / rms {worst:.3e}"
    return rel, worst


@pytest.mark.parametrize("tokens,hidden,inter,experts,topk,skew", [
    (37, 512, 256, 8, 2, False),
    (1, 512, 256, 8, 2, False),          # a single token
    (200, 256, 512, 16, 6, False),       # top-6 as in the benchmark layer
    (300, 512, 256, 8, 2, True),         # skewed routing: one expert spans several 128-row blocks, others empty
])
@pytest.mark.parametrize("fused,block_rows", [(True, 128), (False, 128), (True, 256), (False, 256)])
def test_layer_against_oracle(g, tokens, hidden, inter, experts, topk, skew, fused, block_rows):
    x, logits, w1, w2 = make_layer(tokens + hidden, tokens, hidden, inter, experts, topk, skew)
    ids, wts = g.route(logits, topk)
    layer = g.Nvfp4MoE(w1, w2, experts, topk, clamp=10.0, max_tokens=max(tokens, 64), fused=fused, block_rows=block_rows)
    y = layer(x, ids, wts).clone()
    torch.cuda.synchronize()
    assert_layer_close(y, oracle_layer(x, ids, wts, w1, w2, 10.0), f"T={tokens} H={hidden} I={inter} E={experts} k={topk}")
    # changed inputs through the same object: nothing stale may survive (routes, counts, pool contents)
    x2 = torch.roll(x, 1, dims=0) * 0.5
    ids2, wts2 = g.route(torch.roll(logits, 3, dims=1), topk)
    y2 = layer(x2, ids2, wts2).clone()
    assert_layer_close(y2, oracle_layer(x2, ids2, wts2, w1, w2, 10.0), "second call with changed inputs")
    layer.close()


def test_fused_and_unfused_first_gemm_agree(g):
    # the fused epilogue (SwiGLU + re-quantise inside FC1) must produce the activation bytes of the
    # separate kernel, up to code flips from FP32 summation-order differences in single elements
    tokens, hidden, inter, experts, topk = 200, 512, 512, 4, 2
    x, logits, w1, w2 = make_layer(77, tokens, hidden, inter, experts, topk)
    ids, wts = g.route(logits, topk)
    acts = []
    for fused in (True, False):
        layer = g.Nvfp4MoE(w1, w2, experts, topk, max_tokens=256, fused=fused)
        layer(x, ids, wts)
        torch.cuda.synchronize()
        rows = int(layer.totals[1].item())
        acts.append((to_np(layer.act_packed[:rows]).copy(),
                     O.unpack_scales_u8(to_np(layer.act_scales), layer.pool_rows, inter)[:rows].copy(),
                     to_np(layer.pool_weight[:rows]).copy()))
        layer.close()
    # the padding rows behind an expert's real rows (route weight 0) are written by neither route
    acts = [tuple(a[w != 0] for a in (p, sc, w)) for p, sc, w in acts]
    (pf, sf, wf), (pu, su, wu) = acts
    assert len(wf) == tokens * topk
    # rows land in an arbitrary order inside an expert's group: match them through the route weight
    order_f, order_u = np.argsort(wf, kind="stable"), np.argsort(wu, kind="stable")
    assert np.array_equal(wf[order_f], wu[order_u])
    same_scale = (sf[order_f] == su[order_u]).mean()
    same_code = (pf[order_f] == pu[order_u]).mean()
    assert same_scale > 0.999 and same_code > 0.999, (same_scale, same_code)


def test_second_gemm_scatter_epilogue_exact(g):
    # FC2 fused with the combine: each pool row must land, bit for bit, in the slot its destination code names
    # (here two buffers of this GPU stand in for two ranks), and padding rows (code 0) must write nothing
    import ctypes
    from gpu_kernels_b200 import _lib
    tokens, hidden, inter, experts, topk = 300, 512, 256, 4, 2
    x, logits, w1, w2 = make_layer(5, tokens, hidden, inter, experts, topk)
    ids, wts = g.route(logits, topk)
    for block_rows in (128, 256):
        layer = g.Nvfp4MoE(w1, w2, experts, topk, max_tokens=512, block_rows=block_rows)
        layer(x, ids, wts)
        torch.cuda.synchronize()
        rows = int(layer.totals[1].item())
        weight = layer.pool_weight[:rows].cpu().numpy()
        real = np.flatnonzero(weight != 0)
        rng = np.random.default_rng(block_rows)
        slot_rows = len(real)
        slot_of = rng.permutation(slot_rows)
        owner = rng.integers(0, 2, slot_rows)
        codes = np.zeros(layer.pool_rows, np.int32)
        codes[real] = (owner << 24) | (slot_of + 1)
        row_dst = torch.from_numpy(codes).cuda()
        slots = [torch.full((slot_rows, hidden), -7.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        table = torch.tensor([t.data_ptr() for t in slots], dtype=torch.int64, device="cuda")
        fc2 = layer._plans[block_rows][1]
        _lib.check(_lib.load().gpu_kernels_nvfp4_grouped_run_scatter(
            fc2, row_dst.data_ptr(), table.data_ptr(), slots[0].data_ptr(), 2, slot_rows, 1,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        torch.cuda.synchronize()
        assert _lib.load().gpu_kernels_nvfp4_validate(None) == 0
        expect = [np.full((slot_rows, hidden), -7.0, np.float32) for _ in range(2)]
        pool = layer.out_pool.float().cpu().numpy()
        for r, o, sl in zip(real, owner, slot_of):
            expect[o][sl] = pool[r]
        for o in range(2):
            assert np.array_equal(slots[o].float().cpu().numpy(), expect[o]), (block_rows, o)
        # a destination outside the buffer is skipped and reported, not written
        codes[real[0]] = slot_rows + 1
        row_dst.copy_(torch.from_numpy(codes))
        _lib.load().gpu_kernels_nvfp4_grouped_run_scatter(
            fc2, row_dst.data_ptr(), table.data_ptr(), slots[0].data_ptr(), 2, slot_rows, 1,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert _lib.load().gpu_kernels_nvfp4_validate(None) != 0
        layer.close()


def test_captured_forward_replays_exactly(g):
    # the whole forward as one CUDA graph: replays on new inputs must give the bits of the eager call
    tokens, hidden, inter, experts, topk = 96, 512, 256, 8, 2
    x, logits, w1, w2 = make_layer(11, tokens, hidden, inter, experts, topk)
    layer = g.Nvfp4MoE(w1, w2, experts, topk, max_tokens=128)
    gx, gids, gwts, gy, graph = layer.capture(tokens)
    for seed in (1, 2, 3):
        x, logits, _, _ = make_layer(seed, tokens, hidden, inter, experts, topk)
        ids, wts = g.route(logits, topk)
        eager = layer(x, ids, wts).clone()
        gx.copy_(x); gids.copy_(ids); gwts.copy_(wts)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(gy, eager), seed
    layer.check()
    del graph
    layer.close()
    small = g.Nvfp4MoE(w1, w2, experts, topk, max_tokens=128, pool_rows=512)
    with pytest.raises(RuntimeError):
        small.capture(tokens)
    small.close()


def test_fused_dispatch_matches_quantise_then_pack(g):
    # tokens quantised inside the dispatch kernel (one CTA per token) against the stand-alone quantiser
    # followed by the pack kernel: the same pool rows, hence the same output bits
    for tokens, hidden, inter, experts, topk, skew in ((300, 512, 256, 8, 2, False), (64, 1024, 256, 16, 6, True), (1, 512, 256, 4, 2, False)):
        x, logits, w1, w2 = make_layer(21 + tokens, tokens, hidden, inter, experts, topk, skew)
        ids, wts = g.route(logits, topk)
        outs, pools = [], []
        for fused_dispatch in (True, False):
            layer = g.Nvfp4MoE(w1, w2, experts, topk, max_tokens=512, fused_dispatch=fused_dispatch)
            outs.append(layer(x, ids, wts).clone())
            torch.cuda.synchronize()
            rows = int(layer.totals[1].item())
            weight = layer.pool_weight[:rows].cpu().numpy()
            order = np.lexsort((to_np(layer.pool_packed[:rows]).view(np.uint8)[:, 0], weight))
            pools.append((to_np(layer.pool_packed[:rows])[order], O.unpack_scales_u8(to_np(layer.pool_scales), layer.pool_rows, hidden)[:rows][order], weight[order]))
            layer.check()
            layer.close()
        assert torch.equal(outs[0], outs[1]), (tokens, hidden)
        # the pools hold the same rows (the order inside an expert's group is arrival order)
        assert np.array_equal(pools[0][2], pools[1][2])
        real = pools[0][2] != 0
        assert np.array_equal(pools[0][1][real], pools[1][1][real])


@pytest.mark.parametrize("world,experts,block_rows", [(2, 8, 128), (4, 32, 256), (8, 256, 128)])
def test_plan_agrees_across_ranks_on_pool_rows(g, world, experts, block_rows):
    # every rank derives, from the same gathered counts, where ITS rows start in the pool of each expert's
    # owner (peer_to_pool) and, as an owner, where every source's rows start in its own pool: the two must
    # be the same numbers, or a dispatched row would land in another route's place
    import ctypes
    from gpu_kernels_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(world * 1000 + experts)
    counts = rng.integers(0, 300, size=(world, experts)).astype(np.int32)
    counts[rng.random((world, experts)) < 0.3] = 0                         # empty groups
    local = experts // world
    dev = lambda a: torch.from_numpy(a).cuda()
    matrix = dev(counts)
    capacity = int(((counts.sum(0) + block_rows - 1) // block_rows * block_rows).reshape(world, local).sum(1).max())
    capacity = -(-capacity // 256) * 256
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    peer_offsets, seg_pools = [], []
    for rank in range(world):
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device="cuda")
        send_offset, seg_src, seg_pool = i32(experts + 1), i32(experts + 1), i32(experts)
        block_expert, num_blocks, totals, peer_offset, cursor = i32(capacity // 128), i32(1), i32(4), i32(experts), i32(experts)
        block_valid = i32(capacity // 128)
        _lib.check(lib.gpu_kernels_nvfp4_moe_plan(
            matrix.data_ptr(), world, rank, experts, capacity, block_rows, send_offset.data_ptr(), seg_src.data_ptr(),
            seg_pool.data_ptr(), block_expert.data_ptr(), num_blocks.data_ptr(), totals.data_ptr(), peer_offset.data_ptr(),
            1, cursor.data_ptr(), block_valid.data_ptr(), stream))
        torch.cuda.synchronize()
        assert int(totals[2].item()) == 0
        # real rows per live block: an expert's rows fill its blocks from the front
        live = int(num_blocks.item())
        owned = to_np(matrix).reshape(world, experts)[:, rank * local:(rank + 1) * local].sum(axis=0)
        want_valid = []
        for e in range(local):
            left = int(owned[e])
            for _ in range(-(-left // block_rows)):
                want_valid.append(min(block_rows, left))
                left -= block_rows
        assert to_np(block_valid)[:live].tolist() == want_valid
        peer_offsets.append(to_np(peer_offset))
        seg_pools.append(to_np(seg_pool).reshape(world, local))            # [source rank, local expert] on this owner
    for src in range(world):
        for ge in range(experts):
            owner, e = divmod(ge, local)
            assert peer_offsets[src][ge] == seg_pools[owner][src, e], (src, ge)
    # and the owner's layout is the padded expert-major one
    for owner in range(world):
        padded = (counts[:, owner * local:(owner + 1) * local].sum(0) + block_rows - 1) // block_rows * block_rows
        starts = np.concatenate(([0], np.cumsum(padded)[:-1]))
        assert np.array_equal(seg_pools[owner][0], starts)


def test_routing_plan_pack_unpack_exact(g):
    tokens, hidden, inter, experts, topk = 150, 512, 256, 8, 3
    x, logits, w1, w2 = make_layer(5, tokens, hidden, inter, experts, topk, skew=True)
    ids, wts = g.route(logits, topk)
    layer = g.Nvfp4MoE(w1, w2, experts, topk, max_tokens=256, block_rows=128)
    layer(x, ids, wts)
    torch.cuda.synchronize()
    ids_np, w_np = to_np(ids), to_np(wts)
    counts = np.bincount(ids_np.reshape(-1), minlength=experts)
    assert np.array_equal(to_np(layer.counts_matrix[0]), counts)
    # plan: expert-major pool, each expert padded to 128 rows
    padded = (counts + 127) // 128 * 128
    assert int(layer.num_blocks.item()) == padded.sum() // 128
    expect_blocks = np.repeat(np.arange(experts), padded // 128)
    assert np.array_equal(to_np(layer.block_expert)[:len(expect_blocks)], expect_blocks)
    totals = to_np(layer.totals)
    assert totals[0] == tokens * topk and totals[1] == padded.sum() and totals[2] == 0
    # the pool holds, per expert, exactly the quantised rows (and weights) of the tokens routed to it
    xp = np.zeros((256, hidden), dtype=np.float32)
    xp[:tokens] = to_np(x.float())
    xq, xs = O.quantize(xp)
    xs_rows = O.unpack_scales_u8(xs, 256, hidden)
    pool_q = to_np(layer.pool_packed)
    pool_s = O.unpack_scales_u8(to_np(layer.pool_scales), layer.pool_rows, hidden)
    pool_w = to_np(layer.pool_weight)
    start = np.concatenate(([0], np.cumsum(padded)))
    for e in range(experts):
        tok, choice = np.nonzero(ids_np == e)
        got = slice(start[e], start[e] + counts[e])
        key = lambda q, s, w: sorted(zip(map(bytes, q), map(bytes, s), w.tolist()))
        assert key(pool_q[got], pool_s[got], pool_w[got]) == key(xq[tok], xs_rows[tok], w_np[tok, choice])
        pad = slice(start[e] + counts[e], start[e + 1])
        assert not pool_s[pad].any() and not pool_w[pad].any()          # padding rows carry zero scales
    layer.close()


def test_reduce_order_exact(g):
    # y[t] = bf16(((r0 + r1) + r2) ...) in FP32: bit-exact against the same sequential sum
    from gpu_kernels_b200 import _lib
    tokens, topk, hidden = 9, 6, 512
    gen = torch.Generator(device="cuda").manual_seed(1)
    rows = torch.randn((tokens * topk, hidden), generator=gen, device="cuda").bfloat16()
    pos = torch.randperm(tokens * topk, generator=gen, device="cuda").to(torch.int32)
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device="cuda")
    _lib.check(_lib.load().gpu_kernels_nvfp4_moe_reduce(rows.data_ptr(), pos.data_ptr(), tokens, topk, hidden,
                                                        y.data_ptr(), None, 0, torch.cuda.current_stream().cuda_stream))
    r = to_np(rows.float())[to_np(pos).astype(np.int64)].reshape(tokens, topk, hidden)
    acc = np.zeros((tokens, hidden), dtype=np.float32)
    for j in range(topk):
        acc = (acc + r[:, j]).astype(np.float32)
    assert np.array_equal(to_np(y.float()), MO.round_bf16(acc))


@pytest.mark.parametrize("fused_dispatch", [True, False])
def test_dropped_routes_add_nothing(g, fused_dispatch):
    # an id outside [0, experts) (a router's "dropped" mark) takes no row and adds nothing: the result equals the
    # oracle's with that route removed; nothing is read or written out of bounds and no error is reported
    tokens, hidden, inter, experts, topk = 40, 512, 256, 8, 2
    x, logits, w1, w2 = make_layer(77, tokens, hidden, inter, experts, topk)
    ids, wts = g.route(logits, topk)
    ids = ids.clone()
    ids[3, 0] = -1
    ids[17, 1] = experts
    ids[39, 0] = -7
    ids[39, 1] = 1 << 40
    layer = g.Nvfp4MoE(w1, w2, experts, topk, clamp=10.0, max_tokens=64, fused_dispatch=fused_dispatch)
    for _ in range(2):                                       # the second call must not see rows of the first
        y = layer(x, ids, wts).clone()
        torch.cuda.synchronize()
    layer.check()
    ids_ref = to_np(ids).copy()
    ids_ref[(ids_ref < 0) | (ids_ref >= experts)] = -1
    w1n, w2n = to_np(w1.float()), to_np(w2.float())
    ref = MO.moe_forward_nvfp4_experts(
        to_np(x.float()), ids_ref, to_np(wts),
        lambda e: (MO._quant_dequant_rows(w1n[e]), MO._quant_dequant_rows(w2n[e])), 10.0)
    assert_layer_close(y, ref, "dropped routes")
    assert not to_np(y.float())[39].any()                    # both routes of this token were dropped
    layer.close()


def test_pool_overflow_is_reported(g):
    x, logits, w1, w2 = make_layer(3, 64, 256, 256, 4, 2)
    ids, wts = g.route(logits, 2)
    layer = g.Nvfp4MoE(w1, w2, 4, 2, max_tokens=64, pool_rows=256)
    with pytest.raises(RuntimeError, match="overflow"):
        layer(x, ids, wts)
    layer.close()


@pytest.mark.parametrize("block_rows", [128, 256])
def test_plain_second_gemm_writes_only_the_real_rows(g, block_rows):
    # with the plan's rows-per-block table the output pool gets its real rows, bit-equal to the launch that writes
    # every row, and the padding behind them keeps what was there
    import ctypes
    from gpu_kernels_b200 import _lib
    lib = _lib.load()
    tokens, hidden, inter, experts, topk = 150, 512, 256, 8, 2
    x, logits, w1, w2 = make_layer(9, tokens, hidden, inter, experts, topk, skew=True)
    ids, wts = g.route(logits, topk)
    layer = g.Nvfp4MoE(w1, w2, experts, topk, max_tokens=256, block_rows=block_rows)
    layer(x, ids, wts)
    torch.cuda.synchronize()
    rows = int(layer.totals[1].item())
    real = layer.pool_weight[:rows] != 0
    assert int(real.sum()) == tokens * topk and rows > tokens * topk
    fc2 = layer._plans[block_rows][1]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = []
    for table in (None, layer.block_valid.data_ptr()):
        _lib.check(lib.gpu_kernels_nvfp4_grouped_set_valid_rows(fc2, table))
        layer.out_pool.fill_(-3.0)
        _lib.check(lib.gpu_kernels_nvfp4_grouped_run(fc2, layer.out_pool.data_ptr(), 1, stream))
        torch.cuda.synchronize()
        outs.append(layer.out_pool[:rows].clone())
    everything, masked = outs
    assert torch.equal(masked[real], everything[real])
    assert bool((masked[~real] == -3.0).all()) and not bool((everything[~real] == -3.0).all())
    assert lib.gpu_kernels_nvfp4_validate(None) == 0
    layer.close()


@pytest.mark.parametrize("fused,block_rows", [(True, 128), (False, 128), (True, 256), (False, 256)])
def test_nothing_the_layer_reads_is_left_over_from_before(g, fused, block_rows):
    # every data buffer of the layer is filled with NaN patterns before each call (padding rows are not written any
    # more, so whatever they hold must never reach a real row), a large batch first, then a small one whose padding
    # lies where the large one had real rows
    hidden, inter, experts, topk = 512, 256, 8, 2
    x, logits, w1, w2 = make_layer(31, 300, hidden, inter, experts, topk)
    layer = g.Nvfp4MoE(w1, w2, experts, topk, clamp=10.0, max_tokens=300, fused=fused, block_rows=block_rows)

    def poison():
        for name in ("pool_packed", "pool_scales", "act_packed", "act_scales"):
            getattr(layer, name).fill_(0xFF)
        for name in ("pool_weight", "gate_up", "out_pool", "y"):
            getattr(layer, name).fill_(float("nan"))
        layer.send_pos.fill_(2 ** 30)

    for tokens in (300, 37, 1, 170):
        ids, wts = g.route(logits[:tokens], topk)
        poison()
        y = layer(x[:tokens], ids, wts).clone()
        torch.cuda.synchronize()
        layer.check()
        assert_layer_close(y, oracle_layer(x[:tokens], ids, wts, w1, w2, 10.0), f"poisoned buffers, T={tokens}")
    layer.close()
