"""GPU parity of the gate/up GEMM with the fused SwiGLU epilogue (through the C ABI).

The fused kernel is checked against the unfused pair it replaces - the library's own bf16 GEMM over the fused
gate/up weight, which the other GPU tests pin to the oracle, followed by the CPU restatement of
gk_silu_and_mul_bf16_v1 - and end to end against the oracle's bf16 GEMM result followed by the same restatement.
"""

import numpy as np
import pytest
import torch

from oracle import block_fp8_ref, swiglu_ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gk():
    import gaudi_kernels_b200 as g
    from gaudi_kernels_b200 import _lib
    _lib.load()
    return g


def _problem(m, k, inter, seed, bias):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((m, k), generator=g) * 1.5).to(torch.bfloat16)
    w = torch.randn((2 * inter, k), generator=g) * 0.05
    grid = (2 * inter // 128, (k + 127) // 128)
    s = torch.rand(grid, generator=g) * 2e-3 + 5e-4
    # quantize the fp32 weight block by block into OCP codes the way a checkpoint holds them
    kp = grid[1] * 128
    wp = torch.nn.functional.pad(w, (0, kp - k))
    q = (wp.view(grid[0], 128, grid[1], 128) / s.view(grid[0], 1, grid[1], 1)).clamp(-448, 448)
    codes = q.view(2 * inter, kp)[:, :k].contiguous().to(torch.float8_e4m3fn)
    b = (torch.randn(2 * inter, generator=g) * 0.3) if bias else None
    return x, codes, s, b


def _bf16_step(t):
    """Spacing of bf16 numbers at |t| (t is bf16)."""
    a = t.float().abs().clamp_min(2.0 ** -126)
    return torch.exp2(torch.floor(torch.log2(a)) - 7).double()


@pytest.mark.parametrize("inter,k", [(128, 128), (256, 1040), (1024, 512)])
def test_interleave_is_the_documented_row_order(gk, inter, k):
    rng = np.random.default_rng(inter + k)
    w = rng.integers(0, 256, size=(2 * inter, k), dtype=np.uint8)
    w[w == 0x7f] = 0x7e
    w[w == 0xff] = 0xfe
    s = np.ones((2 * inter // 128, (k + 127) // 128), dtype=np.float32)
    got, s_out = gk.prepare_weight_swiglu(torch.from_numpy(w).cuda(), torch.from_numpy(s).cuda(), native_half=False)
    assert torch.equal(s_out.cpu(), torch.from_numpy(s))
    assert np.array_equal(got.view(torch.uint8).cpu().numpy()[:, :k], swiglu_ref.interleave_gate_up(w))


@pytest.mark.parametrize("m,k,inter,bias", [(1, 128, 128, False), (37, 384, 256, True), (130, 208, 384, False),
                                            (256, 1024, 1024, True), (300, 1000, 512, True), (2048, 512, 2048, False)])
@pytest.mark.parametrize("half", [True, False])
def test_fused_swiglu_matches_gemm_then_silu_and_mul(gk, m, k, inter, bias, half):
    x, codes, s, b = _problem(m, k, inter, seed=m * 7 + inter + k, bias=bias)
    xd = x.cuda()
    a_codes, a_scales = gk.quantize_act_1x128(xd, native_half=half)
    # the unfused pair: bf16 GEMM over the fused weight, then the restated silu_and_mul
    w_plain, s_plain = gk.prepare_weight(codes.cuda(), s.cuda(), native_half=half)
    bd = None if b is None else b.cuda()
    gate_up = gk.gemm_block_fp8(a_codes, a_scales, w_plain, s_plain, bias=bd, schedule=1).cpu()
    want = swiglu_ref.silu_and_mul_bf16(gate_up)
    w_il, s_il = gk.prepare_weight_swiglu(codes.cuda(), s.cuda(), native_half=half)
    got = gk.gemm_block_fp8_swiglu(a_codes, a_scales, w_il, s_il, bias=bd).cpu()
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == (m, inter)
    # same accumulation and the same bf16 rounding of both factors: only the last bit of the product may differ
    diff = (got.double() - want.double()).abs()
    assert bool((diff <= _bf16_step(want) + 1e-36).all()), float((diff - _bf16_step(want)).max())
    # what is left is the error of ex2.approx inside exp(-g): fewer than 1 product in 10 000 lands on the other side
    # of a bf16 rounding boundary (measured 5e-7 .. 6e-5 depending on the spread of the gate values)
    assert float((got != want).float().mean()) < 5e-4
    # end to end against the oracle's GEMM followed by the same step: the GEMM's tolerance (1e-2 of the RMS
    # before rounding, here on each factor) plus the bf16 steps the two roundings can move a product by
    y64, ybf = block_fp8_ref.reference_rows(x, codes, s, native_half=half, bias=b)
    want2 = swiglu_ref.silu_and_mul_bf16(ybf)
    rms = float(want2.double().pow(2).mean().sqrt())
    diff2 = (got.double() - want2.double()).abs()
    assert bool((diff2 <= 3e-2 * rms + 3.0 * _bf16_step(want2)).all()), float(diff2.max())


def test_silu_special_values(gk):
    """g <= -88 gives exactly 0; large positive g passes through; rows beyond M are not written."""
    m, k, inter = 5, 128, 128
    x = torch.zeros((m, k), dtype=torch.bfloat16)
    x[:, 0] = torch.tensor([1.0, -1.0, 0.5, -0.5, 0.0]).to(torch.bfloat16)
    w = torch.zeros((2 * inter, k))
    w[:inter, 0] = torch.linspace(-448, 448, inter)
    w[inter:, 0] = 1.0
    codes = w.to(torch.float8_e4m3fn)
    s = torch.full((2, 1), 0.5)
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    w_il, s_il = gk.prepare_weight_swiglu(codes.cuda(), s.cuda(), native_half=True)
    canvas = torch.full((m + 3, inter), 7.0, dtype=torch.bfloat16, device="cuda")
    got = gk.gemm_block_fp8_swiglu(a_codes, a_scales, w_il, s_il, out=canvas[:m]).cpu()
    assert bool((canvas[m:] == 7.0).all())
    y64, ybf = block_fp8_ref.reference_rows(x, codes, s, native_half=True)
    want = swiglu_ref.silu_and_mul_bf16(ybf)
    assert float(ybf[:, :inter].min()) <= -88.0 and float(ybf[:, :inter].max()) >= 88.0
    diff = (got.double() - want.double()).abs()
    assert bool((diff <= _bf16_step(want) + 1e-36).all())
    assert bool((got[ybf[:, :inter] <= -88.0] == 0).all())


def test_swiglu_rejects_bad_arguments(gk):
    x = torch.zeros((4, 128), dtype=torch.bfloat16, device="cuda")
    a_codes, a_scales = gk.quantize_act_1x128(x, native_half=True)
    w = torch.zeros((192, 128), dtype=torch.uint8, device="cuda")          # I = 96: not a multiple of 128
    with pytest.raises(ValueError):
        gk.prepare_weight_swiglu(w.view(torch.float8_e4m3fn), torch.ones((2, 1), device="cuda"))
    w = torch.zeros((256, 128), dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        gk.gemm_block_fp8_swiglu(a_codes, a_scales, w, torch.ones((3, 1), device="cuda"))
    with pytest.raises(ValueError):
        gk.gemm_block_fp8_swiglu(a_codes, a_scales, w, torch.ones((2, 1), device="cuda"), bias=torch.zeros(100))


@pytest.mark.parametrize("rows,inter", [(1, 14336), (8, 7168), (64, 14336), (5, 100), (3, 7), (2048, 1024)])
def test_standalone_silu_and_mul_matches_restatement(gk, rows, inter):
    g = torch.Generator().manual_seed(rows + inter)
    x = (torch.randn((rows, 2 * inter), generator=g) * 6).to(torch.bfloat16)
    x[0, 0] = -100.0                                   # silu is exactly 0 at and below -88
    x[0, inter] = 3.0
    if inter > 2:
        x[0, 1] = float("nan")                         # NaN gate passes through
        x[0, 2] = 90.0
    want = swiglu_ref.silu_and_mul_bf16(x)
    canvas = torch.full((rows + 1, inter + 8), 7.0, dtype=torch.bfloat16, device="cuda")
    got = gk.silu_and_mul(x.cuda(), out=canvas[:rows, :inter]).cpu()
    assert bool((canvas[rows:] == 7.0).all()) and bool((canvas[:, inter:] == 7.0).all())
    finite = ~torch.isnan(want)
    assert torch.equal(torch.isnan(got), torch.isnan(want))
    diff = (got.double() - want.double()).abs()[finite]
    assert bool((diff <= _bf16_step(want)[finite] + 1e-36).all())
    assert float((got[finite] != want[finite]).float().mean()) < 5e-4 or int((got[finite] != want[finite]).sum()) <= 2
    assert float(got[0, 0]) == 0.0
    # the fused and the stand-alone kernel share the arithmetic: GEMM -> silu_and_mul equals the fused GEMM bit for bit
    if rows == 64:
        m, k, i2 = 64, 512, 256
        xg, codes, s, b = _problem(m, k, i2, seed=3, bias=True)
        a_codes, a_scales = gk.quantize_act_1x128(xg.cuda(), native_half=True)
        w_plain, s_plain = gk.prepare_weight(codes.cuda(), s.cuda(), native_half=True)
        two_step = gk.silu_and_mul(gk.gemm_block_fp8(a_codes, a_scales, w_plain, s_plain, bias=b.cuda(), schedule=1))
        w_il, s_il = gk.prepare_weight_swiglu(codes.cuda(), s.cuda(), native_half=True)
        fused = gk.gemm_block_fp8_swiglu(a_codes, a_scales, w_il, s_il, bias=b.cuda(), small_m=False)   # same schedule as the GEMM above
        assert torch.equal(two_step, fused)


@pytest.mark.parametrize("rows,inter", [(1, 14336), (8, 14336), (64, 1024), (5, 200), (3, 130), (300, 4096)])
@pytest.mark.parametrize("half", [True, False])
def test_fused_silu_quantizer_equals_the_two_kernels(gk, rows, inter, half):
    from oracle import block_fp8_ref
    g = torch.Generator().manual_seed(rows * 3 + inter)
    x = (torch.randn((rows, 2 * inter), generator=g) * 4).to(torch.bfloat16)
    x[0, 0] = -120.0                                    # a product that is exactly zero
    xd = x.cuda()
    h = gk.silu_and_mul(xd)
    want_codes, want_scales = gk.quantize_act_1x128(h, native_half=half)
    codes, scales = gk.silu_quantize_act_1x128(xd, native_half=half)
    assert torch.equal(codes.view(torch.uint8), want_codes.view(torch.uint8))
    assert torch.equal(scales, want_scales)
    # and the pair is the oracle's quantizer applied to the device's bf16 product
    groups = (inter + 127) // 128
    ref_values, ref_scales = block_fp8_ref.quantize_rows(h.cpu(), groups, half)      # values of the codes, [M, G, 128]
    assert torch.equal(codes.cpu().float(), ref_values.reshape(rows, -1)[:, :inter])
    assert torch.equal(scales.cpu(), ref_scales.reshape(rows, groups))


@pytest.mark.parametrize("m,k,inter,bias", [(1, 4096, 14336, False), (8, 4096, 14336, True), (64, 4096, 14336, False),
                                            (32, 2048, 1024, True), (16, 14336, 512, True), (100, 512, 4096, True),
                                            (128, 1024, 2048, False), (5, 384, 128, True)])
def test_decode_bucket_fused_swiglu_equals_gemm_then_silu_and_mul(gk, m, k, inter, bias):
    # the weight-streaming schedule on the interleaved weight (one weight copy for prefill and decode) against the
    # same schedule on the weight in its original order followed by the stand-alone kernel: bit for bit, in the
    # stream-K form (more tiles than SMs), the one-CTA-per-tile form and the cluster form (few tiles)
    x, codes, s, b = _problem(m, k, inter, seed=m * 11 + inter + k, bias=bias)
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    bd = None if b is None else b.cuda()
    w_plain, s_plain = gk.prepare_weight(codes.cuda(), s.cuda(), native_half=True)
    w_il, s_il = gk.prepare_weight_swiglu(codes.cuda(), s.cuda(), native_half=True)
    gate = gk.gemm_block_fp8(a_codes, a_scales, w_plain[:inter], s_plain[:inter // 128], bias=None if bd is None else bd[:inter],
                             schedule=2)
    up = gk.gemm_block_fp8(a_codes, a_scales, w_plain[inter:], s_plain[inter // 128:], bias=None if bd is None else bd[inter:],
                           schedule=2)
    want = gk.silu_and_mul(torch.cat([gate, up], dim=1).contiguous())
    canvas = torch.full((m + 2, inter + 8), 7.0, dtype=torch.bfloat16, device="cuda")
    got = gk.gemm_block_fp8_swiglu(a_codes, a_scales, w_il, s_il, bias=bd, out=canvas[:m, :inter])
    assert bool((canvas[m:] == 7.0).all()) and bool((canvas[:, inter:] == 7.0).all())
    again = gk.gemm_block_fp8_swiglu(a_codes, a_scales, w_il, s_il, bias=bd)
    assert torch.equal(got, again)                                             # counters returned to zero, fixed order
    # the tile decomposition along K is the same when gate and up have as many 128-row tiles together as the
    # interleaved weight has (they always do), so the sums agree exactly where the split points agree; where the
    # stream-K split differs between the two launches the fp32 association differs in the last bits: a factor may
    # then round to the neighbouring bf16 value, which moves the product by up to one step more than its own rounding
    # (and a factor that sits near zero moves by its absolute, not its relative, error: 1e-3 of the RMS covers that)
    slack = 1e-3 * float(want.double().pow(2).mean().sqrt())
    diff = (got.double() - want.double()).abs()
    assert bool((diff <= 3.0 * _bf16_step(want) + slack).all()), float((diff - 3.0 * _bf16_step(want)).max())
    assert float((got != want).float().mean()) < 5e-3
    # and against the large-tile fused kernel on the same interleaved weight
    large = gk.gemm_block_fp8_swiglu(a_codes, a_scales, w_il, s_il, bias=bd, small_m=False)
    diff = (got.double() - large.double()).abs()
    assert bool((diff <= 3.0 * _bf16_step(large) + slack).all()), float((diff - 3.0 * _bf16_step(large)).max())
    assert float((got != large).float().mean()) < 5e-3
    # end to end against the oracle's GEMM followed by the restated step
    y64, ybf = block_fp8_ref.reference_rows(x, codes, s, native_half=True, bias=b)
    want2 = swiglu_ref.silu_and_mul_bf16(ybf)
    rms = float(want2.double().pow(2).mean().sqrt())
    diff2 = (got.double().cpu() - want2.double()).abs()
    assert bool((diff2 <= 3e-2 * rms + 3.0 * _bf16_step(want2)).all()), float(diff2.max())
