"""GPU parity of the block-scaled GEMM (through the C ABI) against the CPU oracle.

Gate (relative tolerance 1e-2): max |y_kernel - y_oracle| / rms(y_oracle) <= 1e-2 on the values
before bf16 rounding (fp32 kernel output against the oracle's FP64 sum).  The bf16 output must equal
the round-to-nearest-even of the kernel's own fp32 output, sit within one bf16 step (plus twice the
pre-rounding error) of the oracle's bf16, and pass the reference's device gate: per-row relative
L2 <= 0.01.
"""

import numpy as np
import pytest
import torch

from oracle import block_fp8_ref, fp8_codec_ref

pytestmark = pytest.mark.gpu

TOL = 1e-2


@pytest.fixture(scope="module")
def gk():
    import gaudi_kernels_b200 as g
    from gaudi_kernels_b200 import _lib
    _lib.load()
    return g


def _case_tensors(c):
    x = torch.from_numpy(c["x_bf16_bits"]).view(torch.bfloat16)
    w = torch.from_numpy(c["w_codes"]).view(torch.float8_e4m3fn)
    s = torch.from_numpy(c["w_scales"])
    b = None if c["bias"] is None else torch.from_numpy(c["bias"])
    return x, w, s, b


def _bf16_step(t):
    """Spacing of bf16 values at |t| (8 significand bits)."""
    a = t.double().abs().clamp_min(2.0 ** -126)
    return torch.exp2(torch.floor(torch.log2(a)) - 7)


def assert_bf16_close(got16, ybf, pre_rounding_err, label=None):
    """bf16 results may differ from the oracle's by one rounding step where the two pre-rounding
    values straddle a rounding boundary; never by more than that plus the pre-rounding error."""
    diff = (got16.double() - ybf.double()).abs()
    bound = _bf16_step(ybf) + 2.0 * pre_rounding_err
    assert bool((diff <= bound).all()), (label, float((diff - bound).max()))


def check_against_oracle(gk, x, w, s, b, half, label, y64=None, ybf=None):
    if y64 is None:
        y64, ybf = block_fp8_ref.reference_rows(x, w, s, native_half=half, bias=b)
    xd, wd, sd = x.cuda(), w.cuda(), s.cuda()
    bd = None if b is None else b.cuda()
    got32 = gk.reference(xd, wd, sd, native_half=half, bias=bd, out_dtype=torch.float32).cpu()
    got16 = gk.reference(xd, wd, sd, native_half=half, bias=bd).cpu()
    assert got16.dtype == torch.bfloat16 and got16.shape == ybf.shape
    rms = float(y64.pow(2).mean().sqrt())
    if rms == 0.0:
        assert not bool(got32.any()) and not bool(got16.any())
        return 0.0
    err = float((got32.double() - y64).abs().max())
    metric = err / rms
    assert metric <= TOL, (label, metric)
    assert torch.equal(got16, got32.to(torch.bfloat16)), label              # same accumulator, RNE
    assert_bf16_close(got16, ybf, err, label)
    num = (got16.double() - ybf.double()).pow(2).sum(1).sqrt()
    den = ybf.double().pow(2).sum(1).sqrt()
    live = den > 0
    assert bool((num[~live] == 0).all()), label                             # identically-zero rows stay zero
    assert bool((num[live] / den[live] <= 0.01).all()), label
    return metric


@pytest.mark.parametrize("half", [False, True])
def test_gemm_matches_reference_fixtures(gk, golden_gemm, gemm_cases, half):
    for name, c in gemm_cases.items():
        x, w, s, b = _case_tensors(c)
        want = torch.from_numpy(golden_gemm[f"{name}.y_bits.half{int(half)}"]).view(torch.bfloat16)
        y64, ybf = block_fp8_ref.reference_rows(x, w, s, native_half=half, bias=b)
        assert torch.equal(ybf, want)
        check_against_oracle(gk, x, w, s, b, half, name, y64, ybf)


def test_host_tensors_round_trip(gk, gemm_cases):
    # the call a CPU user of the reference makes: host tensors in, host bf16 out
    x, w, s, b = _case_tensors(gemm_cases["small_bias"])
    y = gk.reference(x, w, s, native_half=True, bias=b)
    assert y.device.type == "cpu" and y.dtype == torch.bfloat16
    assert torch.equal(y, gk.reference(x.cuda(), w.cuda(), s.cuda(), native_half=True, bias=b.cuda()).cpu())


def test_reference_rejects_nonfinite(gk, gemm_cases):
    x, w, s, b = _case_tensors(gemm_cases["small_bias"])
    bad = x.clone()
    bad[2, 17] = float("inf")
    with pytest.raises(ValueError):
        gk.reference(bad.cuda(), w.cuda(), s.cuda(), native_half=True)
    wb = w.view(torch.uint8).clone()
    wb[5, 5] = 0x7F
    for half in (False, True):
        with pytest.raises(ValueError):
            gk.reference(x.cuda(), wb.view(torch.float8_e4m3fn).cuda(), s.cuda(), native_half=half)
    sb = s.clone()
    sb[0, 0] = -1.0
    with pytest.raises(ValueError):
        gk.reference(x.cuda(), w.cuda(), sb.cuda(), native_half=True)


def _random_problem(m, k, n, seed, bias=False):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).to(torch.bfloat16)
    wf = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    codes, scales = fp8_codec_ref.quantize_block128(wf)
    b = torch.from_numpy(rng.standard_normal(n, dtype=np.float32) * np.float32(0.1)) if bias else None
    return x, torch.from_numpy(codes).view(torch.float8_e4m3fn), torch.from_numpy(scales), b


@pytest.mark.parametrize("m,k,n", [(1, 128, 128), (1, 4096, 512), (8, 1024, 256), (32, 512, 384), (64, 2048, 1024),
                                   (129, 256, 257), (130, 384, 520), (300, 1152, 640), (512, 640, 1032)])
def test_gemm_shapes(gk, m, k, n):
    x, w, s, b = _random_problem(m, k, n, seed=m * 31 + n, bias=(m % 2 == 0))
    check_against_oracle(gk, x, w, s, b, True, (m, k, n))


@pytest.mark.parametrize("m", [1, 8, 32, 64])
def test_gemm_decode_bucket(gk, m):
    # the decode configuration: K=4096, N=14336; both schedules must agree with the oracle,
    # and the weight-streaming schedule must give identical bits whatever the grid size
    k, n = 4096, 14336
    x, w, s, b = _random_problem(m, k, n, seed=100 + m, bias=(m == 8))
    y64, ybf = block_fp8_ref.reference_rows(x, w, s, native_half=True, bias=b)
    rms = float(y64.pow(2).mean().sqrt())
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    wc, ws = gk.prepare_weight(w, s, native_half=True)
    bd = None if b is None else b.cuda()
    outs = {}
    for schedule, cap in ((2, 0), (2, 148), (2, 97), (2, 7), (1, 0)):
        out = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=bd, out_dtype=torch.float32,
                                schedule=schedule, max_ctas=cap)
        err = float((out.double().cpu() - y64).abs().max())
        assert err / rms <= TOL, (schedule, cap, err / rms)
        outs[(schedule, cap)] = out
    again = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=bd, out_dtype=torch.float32, schedule=2, max_ctas=97)
    assert torch.equal(again, outs[(2, 97)])                              # run-to-run identical
    out16 = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=bd)
    assert torch.equal(out16, outs[(2, 0)].to(torch.bfloat16))


@pytest.mark.parametrize("m,k,n", [(3, 384, 130), (17, 1024, 4096), (100, 512, 300), (128, 14336, 512)])
def test_gemm_small_m_ragged(gk, m, k, n):
    x, w, s, b = _random_problem(m, k, n, seed=m + n, bias=True)
    y64, ybf = block_fp8_ref.reference_rows(x, w, s, native_half=True, bias=b)
    rms = float(y64.pow(2).mean().sqrt())
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    wc, ws = gk.prepare_weight(w, s, native_half=True)
    for cap in (0, 5):
        buf = torch.full((m + 2, n + 8), 0.25, dtype=torch.float32, device="cuda")
        out = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=b.cuda(), out=buf[:m, :n], out_dtype=torch.float32,
                                schedule=2, max_ctas=cap)
        assert float((out.double().cpu() - y64).abs().max()) / rms <= TOL
        assert bool((buf[m:] == 0.25).all()) and bool((buf[:, n:] == 0.25).all())


@pytest.mark.parametrize("m,k,n", [(1, 14336, 4096), (64, 14336, 4096), (16, 2048, 2048), (128, 1024, 1024), (5, 384, 9000)])
def test_gemm_small_m_cluster_exchange(gk, m, k, n):
    # few tiles: the CTAs of a tile form a cluster and add their K slices through distributed shared memory
    # (2, 4 or 8 CTAs per tile for these shapes); a caller-imposed CTA limit selects the global-memory form
    x, w, s, b = _random_problem(m, k, n, seed=m * 3 + n, bias=(m > 1))
    y64, ybf = block_fp8_ref.reference_rows(x, w, s, native_half=True, bias=b)
    rms = float(y64.pow(2).mean().sqrt())
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    wc, ws = gk.prepare_weight(w, s, native_half=True)
    bd = None if b is None else b.cuda()
    out = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=bd, out_dtype=torch.float32, schedule=2)
    assert float((out.double().cpu() - y64).abs().max()) / rms <= TOL
    again = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=bd, out_dtype=torch.float32, schedule=2)
    assert torch.equal(out, again)                                         # fixed summation order
    plain = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=bd, out_dtype=torch.float32, schedule=2, max_ctas=148)
    assert float((plain.double().cpu() - y64).abs().max()) / rms <= TOL
    assert float((plain - out).abs().max()) <= 1e-5 * rms + 1e-30       # same K slices up to fp32 association
    out16 = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=bd)
    assert torch.equal(out16, out.to(torch.bfloat16))


def test_gemm_output_tail_is_untouched(gk):
    # sentinel columns right of N and rows below M must survive (out-of-bounds write check)
    m, k, n = 70, 256, 203
    x, w, s, _ = _random_problem(m, k, n, seed=5)
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    wc, ws = gk.prepare_weight(w, s, native_half=True)
    for dtype in (torch.bfloat16, torch.float32):
        buf = torch.full((m + 3, n + 29), 0.5, dtype=dtype, device="cuda")       # row pitch 232: a multiple of 8
        out = buf[:m, :n]
        gk.gemm_block_fp8(a_codes, a_scales, wc, ws, out=out, out_dtype=dtype)
        assert bool((buf[m:, :] == 0.5).all()) and bool((buf[:, n:] == 0.5).all())
        y64, ybf = block_fp8_ref.reference_rows(x, w, s, native_half=True)
        rms = float(y64.pow(2).mean().sqrt())
        if dtype == torch.float32:
            assert float((out.double().cpu() - y64).abs().max()) / rms <= TOL
        else:
            assert_bf16_close(out.cpu(), ybf, 1e-4 * rms)


def test_gemm_many_tiles_persistent_loop(gk):
    # more tiles than SMs, and a grid capped far below the tile count: every CTA walks several tiles
    m, k, n = 1024, 512, 2048
    x, w, s, b = _random_problem(m, k, n, seed=11, bias=True)
    y64, ybf = block_fp8_ref.reference_rows(x, w, s, native_half=True, bias=b)
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    wc, ws = gk.prepare_weight(w, s, native_half=True)
    rms = float(y64.pow(2).mean().sqrt())
    for cap in (0, 5, 1):
        out = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=b.cuda(), out_dtype=torch.float32, max_ctas=cap)
        assert float((out.double().cpu() - y64).abs().max()) / rms <= TOL, cap


@pytest.mark.parametrize("m,k,n", [(256, 256, 256), (300, 384, 520), (1024, 1024, 2048), (130, 208, 257), (512, 640, 1032),
                                   (129, 128, 168), (64, 1152, 3000)])
def test_gemm_pair_schedule_matches_single_cta_schedule(gk, m, k, n):
    # the CTA-pair schedule (cluster of 2, tcgen05 cta_group::2) must reproduce the single-CTA schedule bit for bit
    x, w, s, b = _random_problem(m, k, n, seed=m + k + n, bias=True)
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    wc, ws = gk.prepare_weight(w, s, native_half=True)
    y64, _ = block_fp8_ref.reference_rows(x, w, s, native_half=True, bias=b)
    rms = float(y64.pow(2).mean().sqrt())
    for dtype in (torch.float32, torch.bfloat16):
        one = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=b.cuda(), out_dtype=dtype, schedule=1)
        for sched, cap in ((3, 0), (3, 4), (3, 2)):
            buf = torch.full((m + 1, (n + 7) // 8 * 8 + 8), 3.0, dtype=dtype, device="cuda")
            two = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, bias=b.cuda(), out=buf[:m, :n], out_dtype=dtype,
                                    schedule=sched, max_ctas=cap)
            assert torch.equal(one, two), (dtype, sched, cap)
            assert bool((buf[m:] == 3.0).all()) and bool((buf[:, n:] == 3.0).all())
        if dtype == torch.float32:
            assert float((one.double().cpu() - y64).abs().max()) / rms <= TOL


def test_gemm_prefill_shape_row_sample(gk):
    # the prefill configuration M=8192, K=4096, N=14336 at full size, checked on a seeded sample of rows
    m, k, n = 8192, 4096, 14336
    g = torch.Generator().manual_seed(0)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    wf = (torch.randn((n, k), generator=g) * 0.02).cuda()
    w_ocp, s_ocp = gk.quantize_block128(wf)
    del wf
    wc, ws = gk.prepare_weight(w_ocp, s_ocp, native_half=True)
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    out16 = gk.gemm_block_fp8(a_codes, a_scales, wc, ws)
    out32 = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, out_dtype=torch.float32)
    assert torch.equal(out16, out32.to(torch.bfloat16))
    rows = torch.randperm(m, generator=g)[:48].sort().values
    y64, ybf = block_fp8_ref.reference_rows(x[rows], w_ocp.cpu(), s_ocp.cpu(), native_half=True)
    rms = float(y64.pow(2).mean().sqrt())
    err = float((out32[rows.cuda()].double().cpu() - y64).abs().max())
    assert err / rms <= TOL
    assert_bf16_close(out16[rows.cuda()].cpu(), ybf, err)
    # linearity in the weight scales (size-independent property): doubling every scale doubles the output exactly
    out_2x = gk.gemm_block_fp8(a_codes, a_scales, wc, ws * 2, out_dtype=torch.float32)
    assert torch.equal(out_2x, out32 * 2)


LONG_K_CASES = ("sim_k7168", "sim_k3584", "sim_k22016")


@pytest.mark.parametrize("name", LONG_K_CASES)
def test_gemm_long_k_fixtures_every_schedule(gk, golden_gemm, gemm_cases, name):
    # the long-K shapes of the reference's simulator test (tests/fp8_hybrid_tpcsim_test.cpp:388-392): 56, 28 and 172
    # K blocks per output, where a barrier-phase or scale-prefetch slip of a persistent kernel would show; run
    # through the large-tile, the small-M and the CTA-pair schedules against fixtures the reference produced
    c = gemm_cases[name]
    x, w, s, b = _case_tensors(c)
    for half in (False, True):
        want = torch.from_numpy(golden_gemm[f"{name}.y_bits.half{int(half)}"]).view(torch.bfloat16)
        y64, ybf = block_fp8_ref.reference_rows(x, w, s, native_half=half, bias=b)
        assert torch.equal(ybf, want)
        rms = float(y64.pow(2).mean().sqrt())
        a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=half)
        wc, ws = gk.prepare_weight(w, s, native_half=half)
        outs = {}
        for schedule, cap in ((1, 0), (1, 1), (2, 0), (2, 3), (3, 0)):
            out = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, out_dtype=torch.float32, schedule=schedule, max_ctas=cap)
            err = float((out.double().cpu() - y64).abs().max())
            assert err / rms <= TOL, (name, half, schedule, cap, err / rms)
            out16 = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, schedule=schedule, max_ctas=cap)
            assert torch.equal(out16, out.to(torch.bfloat16))
            assert_bf16_close(out16.cpu(), want, err, (name, half, schedule))
            num = (out16.double().cpu() - want.double()).pow(2).sum(1).sqrt()
            den = want.double().pow(2).sum(1).sqrt()
            assert bool((num[den > 0] / den[den > 0] <= 0.01).all()) and bool((num[den == 0] == 0).all())
            outs[(schedule, cap)] = out
        assert torch.equal(outs[(1, 0)], outs[(1, 1)]) and torch.equal(outs[(1, 0)], outs[(3, 0)])


def _row_sample_check(gk, x, a_codes, a_scales, wc, ws, w_ocp, s_ocp, g, rows=48, **kw):
    """Full-size launch checked on a seeded sample of rows against the oracle; returns the fp32 output."""
    m = x.shape[0]
    out16 = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, **kw)
    out32 = gk.gemm_block_fp8(a_codes, a_scales, wc, ws, out_dtype=torch.float32, **kw)
    assert torch.equal(out16, out32.to(torch.bfloat16))
    pick = torch.randperm(m, generator=g)[:rows].sort().values
    y64, ybf = block_fp8_ref.reference_rows(x[pick], w_ocp.cpu(), s_ocp.cpu(), native_half=True)
    rms = float(y64.pow(2).mean().sqrt())
    err = float((out32[pick.cuda()].double().cpu() - y64).abs().max())
    assert err / rms <= TOL
    assert_bf16_close(out16[pick.cuda()].cpu(), ybf, err)
    num = (out16[pick.cuda()].double().cpu() - ybf.double()).pow(2).sum(1).sqrt()
    assert bool((num / ybf.double().pow(2).sum(1).sqrt() <= 0.01).all())
    return out32


def test_gemm_prefill_down_shape_row_sample(gk):
    # the other prefill shape, M=8192, K=14336, N=4096 (112 K blocks per output), at full size
    m, k, n = 8192, 14336, 4096
    g = torch.Generator().manual_seed(1)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    wf = (torch.randn((n, k), generator=g) * 0.02).cuda()
    w_ocp, s_ocp = gk.quantize_block128(wf)
    del wf
    wc, ws = gk.prepare_weight(w_ocp, s_ocp, native_half=True)
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    out32 = _row_sample_check(gk, x, a_codes, a_scales, wc, ws, w_ocp, s_ocp, g)
    out_2x = gk.gemm_block_fp8(a_codes, a_scales, wc, ws * 2, out_dtype=torch.float32)
    assert torch.equal(out_2x, out32 * 2)


def test_gemm_ffn70b_rank_slice_row_sample(gk):
    # one rank's share of the 8-GPU column-sharded shape: M=16384, K=8192, rank 3's 3584 of N=28672 columns,
    # cut from the full prepared weight by sharded.shard_weight (non-zero row offset into codes and scale grid)
    from gaudi_kernels_b200 import sharded
    m, k, n, world, rank = 16384, 8192, 28672, 8, 3
    g = torch.Generator().manual_seed(2)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    gw = torch.Generator(device="cuda").manual_seed(3)
    w_ocp = torch.empty((n, k), dtype=torch.float8_e4m3fn, device="cuda")
    s_ocp = torch.empty((n // 128, k // 128), dtype=torch.float32, device="cuda")
    for r0 in range(0, n, 3584):                                             # quantized slice by slice to bound fp32 memory
        wf = torch.randn((3584, k), generator=gw, device="cuda") * 0.02
        c, s = gk.quantize_block128(wf)
        w_ocp[r0:r0 + 3584] = c
        s_ocp[r0 // 128:(r0 + 3584) // 128] = s
        del wf
    wc, ws = gk.prepare_weight(w_ocp, s_ocp, native_half=True)
    wl, sl = sharded.shard_weight(wc, ws, world, rank)
    lo, hi = sharded.shard_bounds(n, world, rank)
    assert (lo, hi) == (3 * 3584, 4 * 3584) and wl.data_ptr() == wc.data_ptr() + lo * k
    a_codes, a_scales = gk.quantize_act_1x128(x.cuda(), native_half=True)
    _row_sample_check(gk, x, a_codes, a_scales, wl.contiguous(), sl.contiguous(), w_ocp[lo:hi], s_ocp[lo // 128:hi // 128], g)
    # the views themselves (no copy): what sharded.gemm_sharded is given
    out_view = sharded.gemm_sharded(a_codes, a_scales, wl, sl)
    out_copy = gk.gemm_block_fp8(a_codes, a_scales, wl.contiguous(), sl.contiguous())
    assert torch.equal(out_view, out_copy)

