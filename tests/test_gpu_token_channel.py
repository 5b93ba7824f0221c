"""GPU parity of the per-token / per-channel FP8 variant (through the C ABI) against its CPU restatement."""

import numpy as np
import pytest
import torch

from oracle import fp8_codec_ref, token_channel_ref

pytestmark = pytest.mark.gpu

TOL = 1e-2          # max |y_kernel - y_oracle| / rms(y_oracle) on values before bf16 rounding


@pytest.fixture(scope="module")
def gk():
    import gaudi_kernels_b200 as g
    from gaudi_kernels_b200 import _lib
    _lib.load()
    return g


@pytest.mark.parametrize("shape", [(1, 128), (37, 384), (5, 200), (3, 1000), (64, 4096), (16, 14336), (2, 20480), (7, 130),
                                   # many rows: thread groups of 128, 32, 32, 64, 64, 256 and 256 threads per row
                                   (1024, 4096), (701, 384), (600, 200), (650, 1536), (597, 2048), (600, 8192),
                                   (640, 5000)])
@pytest.mark.parametrize("half", [True, False])
def test_token_quantizer_matches_restatement(gk, shape, half):
    g = torch.Generator().manual_seed(shape[0] * 5 + shape[1])
    x = torch.randn(shape, generator=g) * 3
    if shape[0] > 2:
        x[1] = 0.0                                   # an all-zero row: amax replaced by 1
        x[2] *= 1e-20
    x = x.to(torch.bfloat16)
    want_codes, want_scales = token_channel_ref.quantize_act_token(x.float().numpy(), native_half=half)
    codes, scales = gk.quantize_act_token(x.cuda(), native_half=half)
    assert np.array_equal(scales.cpu().numpy(), want_scales)
    assert np.array_equal(codes.view(torch.uint8).cpu().numpy(), want_codes)
    with pytest.raises(ValueError):
        bad = x.clone()
        bad[0, shape[1] // 2] = float("nan")
        gk.quantize_act_token(bad.cuda(), native_half=half, check_finite=True)


def _weights(n, k, seed):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    amax = np.abs(w).max(axis=1, keepdims=True)
    ws = (amax / np.float32(448.0)).astype(np.float32)
    codes = fp8_codec_ref.half_table()[fp8_codec_ref.cast_e4m3fn_rne((w / ws).astype(np.float32))]
    return codes, (ws.reshape(-1) * np.float32(2.0)).astype(np.float32)


@pytest.mark.parametrize("m,k,n", [(1, 128, 128), (37, 384, 256), (130, 208, 257), (256, 1024, 1024), (300, 1152, 640),
                                   (1024, 512, 2048)])
def test_token_channel_gemm_matches_restatement(gk, m, k, n):
    g = torch.Generator().manual_seed(m + n)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    w_codes, w_scales = _weights(n, k, seed=m * 3 + n)
    bias = (np.arange(n) % 7 - 3).astype(np.float32) * np.float32(0.05) if m % 2 else None
    a_codes, a_scales = gk.quantize_act_token(x.cuda(), native_half=True)
    y64, ybf = token_channel_ref.gemm_token_channel(a_codes.view(torch.uint8).cpu().numpy(), a_scales.cpu().numpy(),
                                                    w_codes, w_scales, bias)
    rms = float(y64.pow(2).mean().sqrt())
    wc = torch.from_numpy(w_codes).cuda()
    ws = torch.from_numpy(w_scales).cuda()
    bd = None if bias is None else torch.from_numpy(bias).cuda()
    for dtype in (torch.float32, torch.bfloat16):
        buf = torch.full((m + 2, (n + 7) // 8 * 8 + 8), 0.75, dtype=dtype, device="cuda")
        out = gk.gemm_token_channel_fp8(a_codes, a_scales, wc, ws, bias=bd, out=buf[:m, :n], out_dtype=dtype)
        assert bool((buf[m:] == 0.75).all()) and bool((buf[:, n:] == 0.75).all())      # nothing written outside
        if dtype == torch.float32:
            got32 = out.clone()
            assert float((out.double().cpu() - y64).abs().max()) / rms <= TOL
        else:
            assert torch.equal(out, got32.to(torch.bfloat16))                          # same accumulator, RNE
            num = (out.double().cpu() - ybf.double()).pow(2).sum(1).sqrt()
            den = ybf.double().pow(2).sum(1).sqrt().clamp_min(1e-30)
            assert bool((num / den <= 0.01).all())          # the reference's device gate, fp8_hybrid_tpcsim_test.cpp:353-379


def test_token_channel_gemm_full_size_linearity(gk):
    # M=8192, K=4096, N=14336 at full size: a seeded row sample against the restatement, and exact linearity in the scales
    m, k, n = 8192, 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w_codes = torch.randint(0, 0x77, (n, k), generator=g, device="cuda", dtype=torch.uint8)
    w_codes |= (torch.randint(0, 2, (n, k), generator=g, device="cuda", dtype=torch.uint8) << 7)
    w_scales = torch.rand(n, generator=g, device="cuda") * 1e-3 + 1e-4
    a_codes, a_scales = gk.quantize_act_token(x, native_half=True)
    out = gk.gemm_token_channel_fp8(a_codes, a_scales, w_codes, w_scales, out_dtype=torch.float32)
    rows = torch.arange(0, m, 171, device="cuda")[:48]
    y64, _ = token_channel_ref.gemm_token_channel(a_codes.view(torch.uint8)[rows].cpu().numpy(), a_scales[rows].cpu().numpy(),
                                                  w_codes.cpu().numpy(), w_scales.cpu().numpy())
    assert float((out[rows].double().cpu() - y64).abs().max()) / float(y64.pow(2).mean().sqrt()) <= TOL
    out2 = gk.gemm_token_channel_fp8(a_codes, a_scales * 2, w_codes, w_scales * 4, out_dtype=torch.float32)
    assert torch.equal(out2, out * 8)
