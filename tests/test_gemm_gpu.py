"""CUDA NVFP4 GEMM through the C ABI against the CPU oracle (small) and the FP32
dequantise-then-matmul path on the GPU (full size).

Acceptance (floating point): relative Frobenius error <= 1e-3 and max abs error
<= 2e-2 x output RMS against the FP32 reference of the same quantised operands.
"""
import os

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from helpers import assert_gemm_close, random_operand, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    import gpu_kernels_b200
    torch.backends.cuda.matmul.allow_tf32 = False
    return gpu_kernels_b200


def nan_output(m, n):
    return torch.full((m, n), float("nan"), device="cuda", dtype=torch.float16)


def run_plan(g, pa, sa, pb, sb, alpha=1.0, variant=None, group_m=None):
    if variant is not None:
        os.environ["NVFP4_B200_VARIANT"] = str(variant)
    try:
        plan = g.Nvfp4Gemm(pa, pb, sa, sb, alpha=alpha)
    finally:
        os.environ.pop("NVFP4_B200_VARIANT", None)
    if group_m is not None:
        plan.set_option("group_m", group_m)
    out = plan.run(nan_output(pa.shape[0], pb.shape[0]))
    plan.validate()
    info = plan.info()
    plan.close()
    return out, info


def test_golden_cfg0(g, golden):
    f = golden("cfg0_256.npz")
    pa, sa, pb, sb = (torch.from_numpy(f[k]).cuda() for k in ("a_packed", "a_scales", "b_packed", "b_scales"))
    out, info = run_plan(g, pa, sa, pb, sb)
    assert info["cta_group"] == 2 and info["tile_n"] == 256
    assert_gemm_close(out, f["c_f32"], "cfg0 vs frozen reference output")
    ref16 = torch.from_numpy(f["c_f16"].view(np.float16).copy())
    # FP16 rounding of nearly equal FP32 sums: the two outputs may differ by one FP16 step on a few elements
    same = (out.cpu() == ref16).float().mean()
    assert same > 0.99, f"only {same:.4f} of FP16 outputs identical to the reference's"
    for variant in (1256, 1128):
        out_v, info_v = run_plan(g, pa, sa, pb, sb, variant=variant)
        assert info_v["cta_group"] == 1
        assert_gemm_close(out_v, f["c_f32"], f"cfg0 variant {variant}")


SHAPES = [
    # (M, N, K, forced variant or None)
    (256, 256, 256, None),          # one stage, one tile
    (256, 256, 512, None),
    (2048, 4096, 2048, None),       # ring wraps, accumulator ping-pong, several tiles per unit
    (128, 512, 1024, None),         # M = 128: single-CTA tiles of 128 x 256
    (128, 384, 512, None),          # N only a multiple of 128: 128 x 128 tiles
    (384, 640, 768, None),
    (512, 256, 4096, None),
    (1024, 1024, 1536, 1256),
    (1024, 1024, 1536, 1128),
    (4096, 2048, 256, None),        # many tiles, single K step: epilogue-bound
]


@pytest.mark.parametrize("m,n,k,variant", SHAPES)
def test_shapes_against_oracle(g, m, n, k, variant):
    a = random_operand(m, k, seed=1 + m + n + k)
    b = random_operand(n, k, seed=2 + m + n + k, scale=0.02)
    pa, sa = g.quantize(a)
    pb, sb = g.quantize(b)
    out, _ = run_plan(g, pa, sa, pb, sb, variant=variant)
    ref = O.gemm_f32(to_np(pa), to_np(sa), to_np(pb), to_np(sb))
    assert_gemm_close(out, ref, f"{m}x{n}x{k}")


K_TAIL_SHAPES = [
    # K is a multiple of 64 but not of the ring's 256: the last ring step reads zero fill beyond K
    (256, 256, 64, None),
    (256, 256, 320, None),
    (128, 512, 1088, None),
    (384, 640, 832, None),
    (2048, 1024, 2240, None),       # ring wraps with a partial last step, K walks that start anywhere
    (512, 512, 1472, 1256),
    (512, 512, 1472, 1128),
]


@pytest.mark.parametrize("m,n,k,variant", K_TAIL_SHAPES)
def test_k_multiple_of_64_against_oracle(g, m, n, k, variant):
    # the reference kernel assumes K % 256 == 0 (kernels/gemm/matmul/sm100.cu:403); its quantiser only needs
    # K % 64 == 0 (reference/python/nvfp4.py:20), which is what this kernel accepts
    a = random_operand(m, k, seed=3 + m + n + k)
    b = random_operand(n, k, seed=4 + m + n + k, scale=0.02)
    pa, sa = g.quantize(a)
    pb, sb = g.quantize(b)
    out, _ = run_plan(g, pa, sa, pb, sb, variant=variant)
    ref = O.gemm_f32(to_np(pa), to_np(sa), to_np(pb), to_np(sb))
    assert_gemm_close(out, ref, f"K tail {m}x{n}x{k}")


@pytest.mark.parametrize("n,k,tiles", [(1280, 1024, 6), (1536, 512, 10), (2304, 2240, 10), (28672, 512, 148)])
def test_ragged_tiles_of_a_single_tile_row(g, n, k, tiles):
    # M = 128: the columns dealt, in units of 64, to `tiles` single-CTA tiles of two widths (256 + 192 or 192 + 128)
    # instead of N / 256 tiles of 256 (N a multiple of 256 here: the plan must be of the 256-column kind). Tile starts that are not multiples of 128 read their scale atoms from a
    # column offset. With every tile walking K from 0 the accumulation order per output is the uniform tiling's:
    # bit-identical; with the default K walk: within the bound.
    m = 128
    pa, sa = g.quantize(random_operand(m, k, seed=400 + n))
    pb, sb = g.quantize(random_operand(n, k, seed=401 + n, scale=0.02))
    ref = g.dequantize(pa, sa) @ g.dequantize(pb, sb).T
    plan = g.Nvfp4Gemm(pa, pb, sa, sb)
    plan.set_option("ragged_tiles", 0)
    plan.set_option("k_skew", 0)
    uniform = plan.run(nan_output(m, n)).clone()
    assert plan.info()["ragged_tiles"] == 0
    try:
        plan.set_option("ragged_tiles", tiles)
    except RuntimeError:
        if tiles > torch.cuda.get_device_properties(0).multi_processor_count:
            pytest.skip("more tiles than this device has SMs")
        raise
    assert plan.info()["ragged_tiles"] == tiles
    ragged = plan.run(nan_output(m, n))
    plan.validate()
    assert not torch.isnan(ragged).any()
    assert torch.equal(ragged, uniform)
    plan.set_option("k_skew", 11)
    assert_gemm_close(plan.run(nan_output(m, n)), ref, f"ragged tiles 128x{n}x{k}")
    for mode in (1, 2):                                     # overlapping launch chains through the ragged route
        plan.set_option("static_operands", mode)
        plan.set_option("k_skew", 0)
        outs = [plan.run(nan_output(m, n)) for _ in range(4)]
        torch.cuda.synchronize()
        assert all(torch.equal(o, uniform) for o in outs)
    plan.validate()
    with pytest.raises(RuntimeError):
        plan.set_option("ragged_tiles", 1)                  # one tile cannot take the whole row
    plan.close()


def test_bf16_output(g):
    # the reference writes FP16 only (include/nvfp4.h:21); "out_bf16" makes the same launch write bfloat16
    for m, n, k in ((256, 512, 1024), (128, 384, 512), (512, 256, 4096)):
        pa, sa = g.quantize(random_operand(m, k, seed=81 + m))
        pb, sb = g.quantize(random_operand(n, k, seed=82 + m, scale=0.02))
        ref = torch.from_numpy(O.gemm_f32(to_np(pa), to_np(sa), to_np(pb), to_np(sb)))
        plan = g.Nvfp4Gemm(pa, pb, sa, sb)
        half = plan.run(nan_output(m, n)).clone()
        plan.set_option("out_bf16", 1)
        assert plan.info()["out_bf16"] == 1
        with pytest.raises(ValueError):
            plan.run(nan_output(m, n))                          # an FP16 tensor is refused now
        out = plan.run(torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16))
        plan.validate()
        assert not torch.isnan(out).any()
        # the same accumulators, rounded to 8 significant bits instead of 11
        want = ref.bfloat16()
        same = (out.cpu() == want).float().mean().item()
        assert same > 0.98, f"{m}x{n}x{k}: only {same:.4f} of the bf16 outputs equal the rounded reference"
        err = (out.float().cpu() - ref).double().norm() / ref.double().norm()
        assert err < 4e-3, err
        plan.set_option("out_bf16", 0)
        assert torch.equal(plan.run(nan_output(m, n)), half)
        plan.close()


def test_l2_side_order_gives_the_same_tiles(g):
    # the L2-side-aware order is a permutation of the tiles: bit-identical C, whatever the census found
    m, n, k = 4096, 8192, 512                                 # 16 x 32 tiles of 256 x 256: more than two per unit
    pa, sa = g.quantize(random_operand(m, k, seed=91))
    pb, sb = g.quantize(random_operand(n, k, seed=92, scale=0.02))
    plan = g.Nvfp4Gemm(pa, pb, sa, sb)
    base = plan.run(nan_output(m, n)).clone()
    try:
        plan.set_option("l2_side", 1)
    except RuntimeError as exc:                              # no two sides found on this device: nothing to compare
        plan.close()
        pytest.skip(str(exc))
    info = plan.info()
    assert info["l2_side"] == 1 and info["side0_units"] + info["side1_units"] == info["units"]
    assert info["side0_units"] > 0 and info["side1_units"] > 0
    for _ in range(3):
        again = plan.run(nan_output(m, n))
        assert torch.equal(again, base)
    plan.validate()
    misses = plan.placement_misses()
    assert 0 <= misses <= 3 * info["units"]
    census = g.gemm.l2_census()
    assert len(census) >= 100 and max(census) > 0
    plan.set_option("l2_side", 0)
    assert plan.info()["l2_side"] == 0
    assert torch.equal(plan.run(nan_output(m, n)), base)
    # a plan whose grid does not fill the GPU is refused
    small = g.Nvfp4Gemm(pa[:256], pb[:256], sa[:256 * k // 16], sb[:256 * k // 16])
    with pytest.raises(RuntimeError):
        small.set_option("l2_side", 1)
    small.close()
    plan.close()


@pytest.mark.parametrize("mode", [1, 2])
def test_overlapping_launches_with_static_operands(g, mode):
    # "static_operands": the caller promises that the kernel in front of a launch does not write B (1) or any
    # operand (2); under programmatic dependent launch the launch then starts while that kernel's last tiles
    # finish, and only its stores of C wait. A chain of launches of two plans with different shapes, each into
    # its own C and, the hard case, all into one shared C (every launch must overwrite the one before it only
    # after that one has finished): bit-identical to ordinary launches.
    specs = [(2048, 1024, 1024), (128, 2560, 2048), (512, 768, 512)]
    plans, wants = [], []
    for i, (m, n, k) in enumerate(specs):
        pa, sa = g.quantize(random_operand(m, k, seed=300 + i))
        pb, sb = g.quantize(random_operand(n, k, seed=310 + i, scale=0.02))
        plan = g.Nvfp4Gemm(pa, pb, sa, sb)
        wants.append(plan.run(nan_output(m, n)).clone())
        plan.set_option("static_operands", mode)
        plans.append(plan)
    torch.cuda.synchronize()
    outs = [nan_output(m, n) for m, n, _ in specs]
    for _ in range(6):
        for plan, out in zip(plans, outs):
            plan.run(out)
    torch.cuda.synchronize()
    for plan, out, want in zip(plans, outs, wants):
        plan.validate()
        assert torch.equal(out, want)
    # one shared output buffer, viewed per shape: the last writer wins, and nothing of an earlier launch lands late
    biggest = max(m * n for m, n, _ in specs)
    shared = torch.full((biggest,), float("nan"), device="cuda", dtype=torch.float16)
    views = [shared[:m * n].view(m, n) for m, n, _ in specs]
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(3):
                for plan, view in zip(plans, views):
                    plan.run(view)
            plans[0].run(views[0])
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        shared.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(views[0], wants[0])
    for plan in plans:
        plan.validate()
        plan.close()


def test_distinct_scale_everywhere(g):
    # every (row, K block) has its own scale byte and codes are random nibbles: a wrong
    # scale column, swizzle or K-slice order cannot cancel out
    m, n, k = 512, 768, 1024
    rng = np.random.default_rng(5)
    pa = rng.integers(0, 256, size=(m, k // 2), dtype=np.uint8)
    pb = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    sa_raw = (40 + (np.arange(m)[:, None] * 7 + np.arange(k // 16)[None, :] * 3) % 24).astype(np.uint8)
    sb_raw = (36 + (np.arange(n)[:, None] * 5 + np.arange(k // 16)[None, :] * 11) % 28).astype(np.uint8)
    sa, sb = O.pack_scales(sa_raw), O.pack_scales(sb_raw)
    ref = O.gemm_f32(pa, sa, pb, sb)
    for variant in (None, 1256, 1128):
        out, _ = run_plan(g, *(torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)), variant=variant)
        assert_gemm_close(out, ref, f"distinct scales, variant {variant}")


def test_alpha_and_group_m(g):
    m, n, k = 1024, 1536, 512
    pa, sa = g.quantize(random_operand(m, k, seed=11))
    pb, sb = g.quantize(random_operand(n, k, seed=12))
    ref = O.gemm_f32(to_np(pa), to_np(sa), to_np(pb), to_np(sb))
    base, _ = run_plan(g, pa, sa, pb, sb)
    assert_gemm_close(base, ref, "alpha 1")
    scaled, _ = run_plan(g, pa, sa, pb, sb, alpha=0.125)
    assert torch.equal(scaled, (base.float() * 0.125).half())       # power of two: exact
    odd, _ = run_plan(g, pa, sa, pb, sb, alpha=0.3)
    assert_gemm_close(odd, ref * np.float32(0.3), "alpha 0.3")
    for gm in (1, 2, 3, 100):
        again, info = run_plan(g, pa, sa, pb, sb, group_m=gm)
        assert torch.equal(again, base), f"tile order group_m={gm} changed the result"


def test_matches_cublaslt(g):
    m = n = k = 1024
    pa, sa = g.quantize(random_operand(m, k, seed=21))
    pb, sb = g.quantize(random_operand(n, k, seed=22))
    ws = torch.empty(32 << 20, dtype=torch.uint8, device="cuda")
    plan = g.Nvfp4Gemm(pa, pb, sa, sb, workspace=ws)
    ours = plan.run(nan_output(m, n))
    theirs = plan.run_cublaslt(nan_output(m, n))
    plan.validate()
    ref = O.gemm_f32(to_np(pa), to_np(sa), to_np(pb), to_np(sb))
    assert_gemm_close(theirs, ref, "cuBLASLt")
    assert_gemm_close(ours, ref, "ours")
    plan.close()


def test_plans_of_different_shapes_interleave(g):
    # per-plan state only: two live plans of different shapes alternate on one stream
    specs = [(256, 512, 512), (1024, 256, 1024)]
    plans, refs = [], []
    for i, (m, n, k) in enumerate(specs):
        pa, sa = g.quantize(random_operand(m, k, seed=31 + i))
        pb, sb = g.quantize(random_operand(n, k, seed=41 + i))
        plans.append(g.Nvfp4Gemm(pa, pb, sa, sb))
        refs.append(O.gemm_f32(to_np(pa), to_np(sa), to_np(pb), to_np(sb)))
    outs = [nan_output(m, n) for m, n, _ in specs]
    for _ in range(3):
        for plan, out in zip(plans, outs):
            plan.run(out)
    for plan, out, ref in zip(plans, outs, refs):
        plan.validate()
        assert_gemm_close(out, ref, "interleaved plans")
        plan.close()


def test_graph_capture_replay(g):
    m = n = k = 512
    pa, sa = g.quantize(random_operand(m, k, seed=51))
    pb, sb = g.quantize(random_operand(n, k, seed=52))
    plan = g.Nvfp4Gemm(pa, pb, sa, sb)
    out = nan_output(m, n)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        plan.run(out)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(4):
                plan.run(out)
        out.fill_(float("nan"))
        graph.replay()
        stream.synchronize()
    plan.validate()
    assert_gemm_close(out, O.gemm_f32(to_np(pa), to_np(sa), to_np(pb), to_np(sb)), "graph replay")
    plan.close()


def test_host_entry_point(g):
    m, n, k = 256, 384, 512
    pa, sa = g.quantize(random_operand(m, k, seed=61))
    pb, sb = g.quantize(random_operand(n, k, seed=62))
    host = [t.cpu().pin_memory() for t in (pa, pb, sa, sb)]
    out = torch.empty((m, n), dtype=torch.float16).pin_memory()
    g.gemm_host(*host, out)
    assert_gemm_close(out, O.gemm_f32(to_np(pa), to_np(sa), to_np(pb), to_np(sb)), "host entry point")


@pytest.mark.parametrize("m,n,k", [(2048, 512, 512), (1024, 384, 768), (4096, 256, 256), (2048, 2048, 512), (1024, 1024, 256)])
def test_host_entry_point_in_row_pieces(g, m, n, k):
    # large M: the host entry point computes and copies back in 4 (or 2) row pieces, and from N = 1024 as many
    # column pieces, on two streams; against
    # one plan over the whole product (tiles start their K walk elsewhere, so single FP16 roundings may
    # differ) and the FP32 reference, also on a second call with other operands
    for seed in (71, 72):
        pa, sa = g.quantize(random_operand(m, k, seed=seed))
        pb, sb = g.quantize(random_operand(n, k, seed=seed + 10, scale=0.02))
        host = [t.cpu().pin_memory() for t in (pa, pb, sa, sb)]
        out = torch.full((m, n), float("nan"), dtype=torch.float16).pin_memory()
        g.gemm_host(*host, out, alpha=0.5)
        whole, _ = run_plan(g, pa, sa, pb, sb, alpha=0.5)
        assert not torch.isnan(out).any()
        assert (out == whole.cpu()).float().mean() > 0.99, (m, n, k, seed)
        assert_gemm_close(out, 0.5 * fp32_reference_on_gpu(g, pa, sa, pb, sb), f"host pieces {m}x{n}x{k}")


def test_argument_errors(g):
    from gpu_kernels_b200._lib import Nvfp4Error
    z = lambda *s: torch.zeros(*s, dtype=torch.uint8, device="cuda")
    with pytest.raises(Nvfp4Error):          # K not a multiple of 64
        g.Nvfp4Gemm(z(128, 48), z(128, 48), z(128 * 6), z(128 * 6))
    with pytest.raises(Nvfp4Error):          # N not a multiple of 8
        g.Nvfp4Gemm(z(128, 128), z(12, 128), z(128 * 16), z(128 * 16))
    with pytest.raises(ValueError):          # scale arrays end in whole atoms
        g.Nvfp4Gemm(z(64, 128), z(128, 128), z(64 * 16), z(128 * 16))
    with pytest.raises(ValueError):
        g.Nvfp4Gemm(z(128, 128), z(128, 256), z(128 * 16), z(128 * 32))


# M any, N any multiple of 8: tiles that reach beyond C (rows >= M, columns >= N are masked in the epilogue; operand
# rows the tensors do not have read as zeros through the tensor maps)
EDGE_SHAPES = [
    (1, 256, 256, 1256), (1, 8, 64, 1128), (7, 136, 128, 1256), (100, 200, 512, 1256), (129, 8, 64, 1128),
    (200, 136, 320, 2256), (300, 1000, 1024, 1256), (500, 1000, 512, 2256), (250, 248, 2240, 2256),
    (128, 4104, 512, 1128), (4097, 264, 256, 1128), (33, 28664, 1024, 1256),
]


@pytest.mark.parametrize("m,n,k,variant", EDGE_SHAPES)
def test_m_and_n_that_are_not_whole_tiles(g, m, n, k, variant):
    a = random_operand(m, k, seed=m + 3 * k)
    b = random_operand(n, k, seed=n + 5 * k, scale=0.05)
    pa, sa = g.quantize(a)
    pb, sb = g.quantize(b)
    # what the scale bytes of the rows beyond M and N hold must not matter: NaN scales there
    sa = sa.clone(); sb = sb.clone()
    ua = g.unpack_scales(sa, -(-m // 128) * 128, k); ua[m:] = 0x7F
    ub = g.unpack_scales(sb, -(-n // 128) * 128, k); ub[n:] = 0x7F
    sa2, sb2 = g.pack_scales(ua), g.pack_scales(ub)
    plan = g.Nvfp4Gemm(pa, pb, sa2, sb2)
    info = plan.info()
    assert info["cta_group"] * 1000 + info["tile_n"] == variant, info
    whole = torch.full((m + 3, n), float("nan"), dtype=torch.float16, device="cuda")
    whole[m:] = 77.0
    out = whole[:m]
    plan.run(out)
    plan.validate()
    ref = O.dequantize_padded(to_np(pa), to_np(sa)) @ O.dequantize_padded(to_np(pb), to_np(sb)).T
    assert_gemm_close(out, ref, f"edge {m}x{n}x{k}")
    assert bool((whole[m:] == 77.0).all()), "rows beyond M were written"
    plan.set_option("out_bf16", 1)
    got = plan.run().float().cpu().numpy()
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 8e-3
    plan.set_option("out_bf16", 0)
    for key in ("split_k",):
        with pytest.raises(Exception):
            plan.set_option(key, 1)
    plan.close()


def test_mxfp4_edge_shapes(g):
    for m, n, k in [(1, 264, 256), (100, 200, 512), (500, 1000, 384)]:
        a = random_operand(m, k, seed=m + k)
        b = random_operand(n, k, seed=n + k, scale=0.05)
        pa, sa = g.quantize_mx(a)
        pb, sb = g.quantize_mx(b)
        plan = g.Nvfp4Gemm(pa, pb, sa, sb, mx=True)
        out = plan.run(torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda"))
        plan.validate()
        ref = (O.dequantize_padded(to_np(pa), to_np(sa), O.dequantize_mx) @
               O.dequantize_padded(to_np(pb), to_np(sb), O.dequantize_mx).T)
        assert_gemm_close(out, ref, f"mxfp4 edge {m}x{n}x{k}")
        plan.close()


def fp32_reference_on_gpu(g, pa, sa, pb, sb):
    """The reference's check (dequantise both operands, FP32 matmul) at full size on the GPU.
    The dequantise kernel is itself pinned bit-exactly to the oracle in test_quantize_gpu.py."""
    return g.dequantize(pa, sa) @ g.dequantize(pb, sb).T


@pytest.mark.parametrize("size", [8192, 16384])
def test_full_size_square(g, size):
    a = random_operand(size, size, seed=0)
    b = random_operand(size, size, seed=1)
    pa, sa = g.quantize(a)
    pb, sb = g.quantize(b)
    del a, b
    out, info = run_plan(g, pa, sa, pb, sb)
    assert info["cta_group"] == 2
    ref = fp32_reference_on_gpu(g, pa, sa, pb, sb)
    assert_gemm_close(out, ref, f"{size}^3 vs FP32 dequantise-then-matmul")
    if size == 8192:
        # 64 sampled rows against the CPU oracle too
        rows = torch.arange(0, size, 128)[:64] + torch.arange(64) % 128
        a_rows = O.dequantize(to_np(pa), to_np(sa))[rows.numpy()]
        b_all = O.dequantize(to_np(pb), to_np(sb))
        assert_gemm_close(out[rows.cuda()], a_rows @ b_all.T, "8192^3 sampled rows vs CPU oracle")


def test_full_size_skinny(g):
    m, n, k = 128, 28672, 8192
    pa, sa = g.quantize(random_operand(m, k, seed=0))
    pb, sb = g.quantize(random_operand(n, k, seed=1, scale=0.02))
    out, info = run_plan(g, pa, sa, pb, sb)
    assert info["cta_group"] == 1
    assert_gemm_close(out, fp32_reference_on_gpu(g, pa, sa, pb, sb), "skinny vs FP32 dequantise-then-matmul")


SPLIT_K_SHAPES = [
    # (M, N, K, S): far fewer tiles than SMs and a long K loop
    (128, 512, 4096, 4),            # 2 tiles: 8 units of 4 ring steps
    (128, 3584, 8192, 4),           # the decode shape's slab on one of eight GPUs
    (256, 256, 8192, 4),            # CTA pairs, one tile
    (512, 512, 4096, 4),            # CTA pairs, 4 tiles
]


@pytest.mark.parametrize("m,n,k,split", SPLIT_K_SHAPES)
def test_split_k_against_whole_tiles(g, m, n, k, split):
    # S units per tile: same result as the unsplit schedule up to FP32 summation order, reproducible from
    # launch to launch (the slices are added in a fixed order), flags lowered again after every launch
    a = random_operand(m, k, seed=11 + m + n + k)
    b = random_operand(n, k, seed=12 + m + n + k, scale=0.02)
    pa, sa = g.quantize(a)
    pb, sb = g.quantize(b)
    plan = g.Nvfp4Gemm(pa, pb, sa, sb)
    assert plan.info()["split_k"] == 0                  # opt-in
    plan.set_option("split_k", 1)
    info = plan.info()
    assert info["split_k"] == split, info
    outs = [plan.run(nan_output(m, n)).clone() for _ in range(3)]
    plan.validate()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    plan.set_option("split_k", 0)
    assert plan.info()["split_k"] == 0 and plan.info()["units"] * split == info["units"]
    whole = plan.run(nan_output(m, n)).clone()
    plan.set_option("split_k", 1)
    again = plan.run(nan_output(m, n))
    plan.validate()
    assert torch.equal(again, outs[0])
    ref = g.dequantize(pa, sa) @ g.dequantize(pb, sb).T
    assert_gemm_close(outs[0], to_np(ref), f"split-K {m}x{n}x{k}")
    assert_gemm_close(whole, to_np(ref), f"whole tiles {m}x{n}x{k}")
    diff = (outs[0].float() - whole.float()).abs().max().item()
    assert diff <= 2e-3 * ref.abs().max().item(), diff
    # inside a CUDA graph, replayed
    graph = torch.cuda.CUDAGraph()
    out = nan_output(m, n)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        plan.run(out)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        plan.run(out)
    for _ in range(2):
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, outs[0])
    plan.validate()
    del graph
    plan.close()


def test_split_k_is_left_off_where_it_cannot_gain(g):
    for m, n, k in ((256, 256, 256), (8192, 8192, 256), (128, 28672, 1024), (384, 640, 2048), (1024, 2048, 4096)):
        a = random_operand(m, k, seed=5)
        b = random_operand(n, k, seed=6, scale=0.02)
        pa, sa = g.quantize(a)
        pb, sb = g.quantize(b)
        plan = g.Nvfp4Gemm(pa, pb, sa, sb)
        assert plan.info()["split_k"] == 0
        with pytest.raises(RuntimeError):
            plan.set_option("split_k", 1)
        plan.close()


@pytest.mark.parametrize("m,n,k,dtype", [(128, 1024, 512, torch.bfloat16), (256, 512, 1024, torch.float16),
                                         (100, 264, 256, torch.float32), (128, 7168, 2048, torch.bfloat16)])
def test_linear_quantises_into_the_plan_and_multiplies(g, m, n, k, dtype):
    # quantise + GEMM chained on the stream (the GEMM starts while the quantiser runs): the plan's A and SFA hold
    # exactly what `quantize` gives, C is bit-equal to the two-call sequence, also when replayed from a graph
    # with other activations each time
    b = random_operand(n, k, seed=9, scale=0.05)
    pb, sb = g.quantize(b)
    pa = torch.zeros((m, k // 2), dtype=torch.uint8, device="cuda")
    sa = torch.zeros(g.nvfp4.scale_rows(m) * k // 16, dtype=torch.uint8, device="cuda")
    plan = g.Nvfp4Gemm(pa, pb, sa, sb)
    xs = [random_operand(m, k, seed=40 + i, dtype=torch.float32).to(dtype) for i in range(3)]
    want = []
    for x in xs:
        qa, qs = g.quantize(x)
        ref_plan = g.Nvfp4Gemm(qa, pb, qs, sb)
        want.append((qa, qs, ref_plan.run().clone()))
        ref_plan.validate()
        ref_plan.close()
    for x, (qa, qs, c) in zip(xs, want):
        out = plan.linear(x)
        plan.validate()
        assert torch.equal(pa, qa) and torch.equal(sa, qs)
        assert torch.equal(out, c)
    x_in = xs[0].clone()
    out = torch.empty((m, n), dtype=torch.float16, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            plan.linear(x_in, out)
            plan.linear(x_in, out)
    torch.cuda.current_stream().wait_stream(side)
    for x, (_, _, c) in zip(xs, want):
        x_in.copy_(x)
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, c)
    plan.validate()
    plan.close()
