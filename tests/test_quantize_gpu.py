"""CUDA quantiser / dequantiser against the oracle and the frozen reference outputs: bit-exact."""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from helpers import bf16_from_bits, random_operand, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    import gpu_kernels_b200
    return gpu_kernels_b200


def check_exact(g, x: torch.Tensor, expect_packed, expect_scales):
    packed, scales = g.quantize(x)
    torch.cuda.synchronize()
    assert np.array_equal(to_np(scales), expect_scales), "scale bytes differ"
    assert np.array_equal(to_np(packed), expect_packed), "packed codes differ"
    return packed, scales


def test_golden_cfg0(g, golden):
    f = golden("cfg0_256.npz")
    for name in ("a", "b"):
        p, s = check_exact(g, bf16_from_bits(f[f"{name}_bf16"]), f[f"{name}_packed"], f[f"{name}_scales"])
    d = g.dequantize(p, s)
    assert np.array_equal(to_np(d), O.dequantize(f["b_packed"], f["b_scales"]))
    pa = torch.from_numpy(f["a_packed"]).cuda()
    sa = torch.from_numpy(f["a_scales"]).cuda()
    assert np.array_equal(to_np(g.dequantize(pa, sa)), f["a_dequant"])


def test_golden_distributions(g, golden):
    f = golden("dists.npz")
    check_exact(g, bf16_from_bits(f["w_bf16"]), f["w_packed"], f["w_scales"])
    check_exact(g, torch.from_numpy(f["f_f32"]).cuda(), f["f_packed"], f["f_scales"])


def test_golden_adversarial(g, golden):
    f = golden("adversarial.npz")
    p, s = check_exact(g, torch.from_numpy(f["x_f32"]).cuda(), f["packed"], f["scales"])
    d = to_np(g.dequantize(p, s))
    assert np.array_equal(np.isnan(d), np.isnan(f["dequant"]))
    assert np.array_equal(np.nan_to_num(d), np.nan_to_num(f["dequant"]))


def test_reference_known_answers(g):
    # tests/test_nvfp4.py:30-35 of the reference, through the CUDA path
    values = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6]).repeat(128, 4).cuda()
    packed, scales = g.quantize(values)
    assert packed[0, :8].tolist() == [0x10, 0x32, 0x54, 0x76, 0x90, 0xBA, 0xDC, 0xFE]
    assert torch.equal(g.dequantize(packed, scales), values)
    # tests/test_nvfp4.py:12-15: every code and every tie, one value per block so the scale is known
    x = torch.zeros(128, 64 * 18)
    probes = [0, .5, 1, 1.5, 2, 3, 4, 6, -.5, -6, .25, .75, 1.25, 1.75, 2.5, 3.5, 5, 100]
    for i, v in enumerate(probes):
        x[:, i * 64 + 1] = v
        x[:, i * 64] = 6.0 if abs(v) <= 6 else 0.0          # pins the scale to 1.0 (except the saturating probe)
    p, s = O.quantize(x.numpy())
    check_exact(g, x.cuda(), p, s)
    codes = p[0, 0::32] >> 4
    assert codes[:17].tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 9, 15, 0, 2, 2, 4, 4, 6, 6]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,k,scale", [(128, 64, 1.0), (256, 192, 0.02), (384, 320, 30.0), (1024, 2048, 1.0),
                                          (128, 8192, 1e-3)])
def test_random_against_oracle(g, dtype, rows, k, scale):
    x = random_operand(rows, k, seed=rows + k, scale=scale, dtype=dtype)
    p, s = O.quantize(to_np(x.float()))
    packed, scales = check_exact(g, x, p, s)
    assert np.array_equal(to_np(g.dequantize(packed, scales)), O.dequantize(p, s))


def _all_scales():
    return O.ue4m3_to_f32(np.arange(1, 0x7F, dtype=np.uint8))          # every finite positive E4M3 value


def test_division_free_path_fp32_neighbourhood_of_every_midpoint(g):
    # The kernel replaces the 16 IEEE divisions by a reciprocal and a residual correction; this is
    # where that could differ from the reference: FP32 values within a few ulps of every midpoint
    # times every possible scale, both signs, with an element 6*s pinning the block scale to s.
    s = _all_scales()                                                # 126 scales
    mids = np.array([.25, .75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    t = (mids[None, :] * s[:, None]).astype(np.float32)             # exact products
    ulps = np.arange(-3, 4)
    probes = (t.view(np.int32)[:, :, None] + ulps[None, None, :].astype(np.int32)).view(np.float32)
    probes = probes.reshape(126, 49)                                  # per scale: 7 midpoints x 7 offsets
    x = np.zeros((128, 126 * 8 * 16), dtype=np.float32)             # per row and scale: 8 blocks of 16
    blocks = x.reshape(128, 126, 8, 16)
    lane = np.arange(14)
    for r in range(128):
        for b in range(8):
            pick = (15 * b + 3 * r + lane) % 49
            sign = np.where((lane + r + b) % 2, -1.0, 1.0).astype(np.float32)
            blocks[r, :, b, 0] = 6.0 * s
            blocks[r, :, b, 1:15] = probes[:, pick] * sign[None, :]
            blocks[r, :, b, 15] = (-1.0 if r % 2 else 1.0) * s * np.float32(2.0 ** -140)   # quotient below the normal range
    p, sc = O.quantize(x)
    assert set(np.unique(O.unpack_scales_u8(sc, 128, x.shape[1]))) == set(range(1, 0x7F))
    check_exact(g, torch.from_numpy(x).cuda(), p, sc)


def test_division_free_path_every_bf16_against_every_scale(g):
    # every non-negative bf16 value up to 8*s (and its negative) beside a 6*s pin, for all 126 scales
    s = _all_scales()
    rows = []
    for sv in s:
        top = np.float32(8.0) * sv
        top_bits = int(np.float32(top).view(np.uint32)) >> 16
        vals = O.bf16_to_f32(np.arange(0, top_bits + 1, dtype=np.uint16))
        vals = np.concatenate((vals, -vals))
        n = -(-len(vals) // 15) * 15
        vals = np.concatenate((vals, np.zeros(n - len(vals), dtype=np.float32))).reshape(-1, 15)
        blk = np.concatenate((np.full((len(vals), 1), 6.0 * sv, dtype=np.float32), vals), axis=1)
        rows.append(blk.reshape(-1))
    flat = np.concatenate(rows)
    k = 4096
    total = -(-len(flat) // (128 * k)) * 128 * k
    x = np.concatenate((flat, np.zeros(total - len(flat), dtype=np.float32))).reshape(-1, k)
    p, sc = O.quantize(x)
    check_exact(g, torch.from_numpy(x).cuda().bfloat16(), p, sc)
    check_exact(g, torch.from_numpy(x).cuda(), p, sc)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_every_16bit_value_as_block_maximum(g, dtype):
    # amax / 6 is computed without a division for 16-bit inputs: every positive pattern (NaNs and
    # infinity included) alone in its block, and again beside smaller neighbours
    bits = np.arange(0x8000, dtype=np.uint16)
    vals = (O.bf16_to_f32(bits) if dtype == torch.bfloat16 else bits.view(np.float16).astype(np.float32))
    x = np.zeros((256, 128 * 16), dtype=np.float32)
    blocks = x.reshape(256, 128, 16)
    blocks[:, :, 5] = vals.reshape(256, 128)
    with np.errstate(invalid="ignore", over="ignore"):
        blocks[:, :, 9] = np.where(np.isfinite(vals), -vals * np.float32(0.4140625), 0).reshape(256, 128)
        blocks[:, :, 12] = np.where(np.isfinite(vals), vals * np.float32(0.2080078125), 0).reshape(256, 128)
    xt = torch.from_numpy(x).cuda().to(dtype)
    p, sc = O.quantize(xt.float().cpu().numpy())
    check_exact(g, xt, p, sc)


def test_every_bf16_value(g):
    # all 65536 bf16 bit patterns (NaNs and infinities included), one per block position in turn
    bits = np.arange(65536, dtype=np.uint16)
    x = np.zeros((128, 65536 // 128 * 16), dtype=np.uint16)         # 512 blocks per row
    x.reshape(128, -1, 16)[:, :, 3] = bits.reshape(128, 512)
    x.reshape(128, -1, 16)[:, :, 7] = 0x3F80                        # a 1.0 beside it
    xt = bf16_from_bits(x)
    p, s = O.quantize(O.bf16_to_f32(x))
    check_exact(g, xt, p, s)


def test_full_size_slabs_match_oracle(g):
    # 8192 x 8192 (the benchmark operand): 128-row slabs are independent, so random slabs pin the whole
    x = random_operand(8192, 8192, seed=0)
    packed, scales = g.quantize(x)
    torch.cuda.synchronize()
    rng = np.random.default_rng(0)
    for blk in rng.choice(64, size=5, replace=False):
        rows = slice(blk * 128, (blk + 1) * 128)
        p, s = O.quantize(to_np(x[rows].float()))
        assert np.array_equal(to_np(packed[rows]), p)
        assert np.array_equal(to_np(scales[blk * 128 * 512:(blk + 1) * 128 * 512]), s)
    # size-independent properties over every element: the scale is the E4M3 rounding of
    # clamp(amax/6), and each code is a nearest E2M1 level of x / scale.
    xf = x.float()
    amax = xf.reshape(8192, -1, 16).abs().amax(-1)
    want_scale = (amax / 6).clamp(min=2 ** -9, max=448).to(torch.float8_e4m3fn)
    got_scale = g.unpack_scales(scales, 8192, 8192)
    assert torch.equal(got_scale, want_scale.view(torch.uint8))
    levels = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6], device="cuda")
    q = (xf.reshape(8192, -1, 16) / want_scale.float()[..., None]).reshape(8192, 8192)
    codes = torch.stack((packed & 15, packed >> 4), dim=-1).reshape(8192, 8192)
    chosen = levels[(codes & 7).long()]
    best = (q.abs()[..., None] - levels).abs().amin(-1)
    assert torch.equal((q.abs() - chosen).abs(), best)
    assert torch.equal((codes >> 3).bool(), q < 0)


def test_shape_errors(g):
    from gpu_kernels_b200._lib import Nvfp4Error
    with pytest.raises(Nvfp4Error):
        g.quantize(torch.zeros(128, 48, device="cuda"))
    with pytest.raises(Nvfp4Error):
        g.quantize(torch.zeros(0, 64, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,k", [(1, 64), (100, 192), (129, 256), (300, 1024), (1000, 320)])
def test_any_row_count(g, dtype, rows, k):
    # the reference's quantiser applied to the tensor with zero rows appended up to whole atoms, bit for bit:
    # packed bytes of the true rows, and every byte of the scale atoms (0x01 for the rows that do not exist)
    x = random_operand(rows, k, seed=rows + k, scale=2.0, dtype=dtype)
    packed, scales = g.quantize(x)
    assert packed.shape == (rows, k // 2) and scales.numel() == -(-rows // 128) * 128 * k // 16
    want_p, want_s = O.quantize_padded(to_np(x.float()))
    assert np.array_equal(to_np(packed), want_p) and np.array_equal(to_np(scales), want_s)
    assert np.array_equal(to_np(g.dequantize(packed, scales)), O.dequantize_padded(want_p, want_s))
    # the scaled and the MXFP4 quantisers follow the same rule
    ps, ss = g.quantize(x, tensor_scale=0.37)
    wp, ws = O.quantize_padded(to_np(x.float()) * np.float32(g.nvfp4.inverse_tensor_scale(0.37)))
    assert np.array_equal(to_np(ps), wp) and np.array_equal(to_np(ss), ws)
    if k % 128 == 0:
        pm, sm = g.quantize_mx(x)
        wp, ws = O.quantize_padded(to_np(x.float()), O.quantize_mx)
        assert np.array_equal(to_np(pm), wp) and np.array_equal(to_np(sm), ws)
        assert np.array_equal(to_np(g.dequantize_mx(pm, sm)), O.dequantize_padded(wp, ws, O.dequantize_mx))


def test_a_partial_last_tile_writes_nothing_beyond_its_rows(g):
    rows, k = 130, 256
    x = random_operand(rows, k, seed=3)
    whole = torch.full((rows + 64, k // 2), 0xEE, dtype=torch.uint8, device="cuda")
    scales = torch.empty(256 * k // 16, dtype=torch.uint8, device="cuda")
    from gpu_kernels_b200 import _lib
    _lib.check(_lib.load().gpu_kernels_nvfp4_quantize(x.data_ptr(), 0, whole.data_ptr(), scales.data_ptr(), rows, k,
                                                     torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert bool((whole[rows:] == 0xEE).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_two_level_scaling_is_bit_exact_and_recovers_the_product(g, dtype):
    # tensor scale gA = amax / (6 * 448): values * float32(1 / gA) quantised by the block rule; bit-exact against the
    # oracle's statement of exactly that, and the GEMM with alpha = gA * gB gives back the unscaled product
    rows, k = 256, 512
    a = (random_operand(rows, k, seed=5, scale=37.0, dtype=torch.float32)).to(dtype)
    b = (random_operand(384, k, seed=6, scale=0.003, dtype=torch.float32)).to(dtype)
    ga, gb = g.nvfp4.tensor_scale_for(a), g.nvfp4.tensor_scale_for(b)
    pa, sa = g.quantize(a, tensor_scale=ga)
    pb, sb = g.quantize(b, tensor_scale=gb)
    for x, scale, p, s in ((a, ga, pa, sa), (b, gb, pb, sb)):
        want_p, want_s = O.quantize_scaled(to_np(x.float()), g.nvfp4.inverse_tensor_scale(scale))
        assert np.array_equal(to_np(s), want_s) and np.array_equal(to_np(p), want_p)
        assert int(to_np(s).max()) >= 0x7E - 8          # the largest block scale sits at the top of the E4M3 range
    plan = g.Nvfp4Gemm(pa, pb, sa, sb, alpha=ga * gb)
    out = plan.run()
    plan.validate()
    ref = to_np(a.float()) @ to_np(b.float()).T
    got = to_np(out.float())
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    assert rel < 0.2, rel                                # FP4 quantisation noise of both operands, not a scaling error
    deq = (O.dequantize(to_np(pa), to_np(sa)) @ O.dequantize(to_np(pb), to_np(sb)).T) * np.float32(ga * gb)
    assert np.linalg.norm(got - deq) / np.linalg.norm(deq) < 2e-3
    plan.close()
    # without the tensor scale the small operand loses its block scales to the E4M3 subnormals
    _, s_plain = g.quantize(b)
    assert int(to_np(s_plain).max()) < int(to_np(sb).max())
