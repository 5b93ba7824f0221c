"""GPU parity of the codec, quantizer and decode kernels (through the C ABI) against the CPU oracle: bit-exact."""

import numpy as np
import pytest
import torch

import cases
from oracle import fp8_codec_ref as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gk():
    import gaudi_kernels_b200 as g
    from gaudi_kernels_b200 import _lib
    _lib.load()
    return g


def _u8(t):
    return t.view(torch.uint8).cpu().numpy()


def _fp8(a, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.float8_e4m3fn).to(device)


def test_reencode_reference_vectors(gk, golden_codec):
    # exhaustive 254-code map, known answer, seeded random - all produced by the reference itself
    for name, (codes, scales) in cases.codec_cases().items():
        for device in ("cuda", "cpu"):
            w = _fp8(codes, device)
            s = torch.from_numpy(scales).to(device)
            before = _u8(w).copy()
            enc, adj, rounded = gk.reencode_e4m3fn_half(w, s)
            assert enc.device.type == device and enc.dtype == torch.float8_e4m3fn and enc.shape == w.shape
            assert np.array_equal(_u8(enc), golden_codec[name + ".encoded"]), name
            assert np.array_equal(adj.cpu().numpy(), golden_codec[name + ".adjusted"]), name
            assert rounded == int(golden_codec[name + ".rounded"]), name
            assert np.array_equal(_u8(w), before)                       # input untouched
    assert int(golden_codec["all_finite.rounded"]) == 16 and int(golden_codec["known.rounded"]) == 1


def test_reencode_rejects_nonfinite_codes_and_bad_scales(gk):
    one = torch.ones(1, device="cuda")
    for code in (0x7F, 0xFF):
        w = _fp8(np.array([0, code], dtype=np.uint8))
        with pytest.raises(ValueError, match="nonfinite"):
            gk.reencode_e4m3fn_half(w, one)
        assert _u8(w).tolist() == [0, code]
    z = _fp8(np.zeros(2, dtype=np.uint8))
    for bad in (float("nan"), float("inf"), -1.0, torch.finfo(torch.float32).max):
        with pytest.raises(ValueError):
            gk.reencode_e4m3fn_half(z, torch.tensor([bad], dtype=torch.float32, device="cuda"))
    # a NaN code deep inside a large buffer, and in the unaligned tail
    big = np.zeros(3 * 1024 * 1024 + 5, dtype=np.uint8)
    for pos in (1234567, big.size - 1):
        b = big.copy()
        b[pos] = 0xFF
        with pytest.raises(ValueError, match="nonfinite"):
            gk.reencode_e4m3fn_half(_fp8(b), one)


@pytest.mark.parametrize("n", [1, 15, 16, 17, 4099, 1 << 20, (1 << 22) + 3])
def test_reencode_ragged_sizes(gk, n):
    rng = np.random.default_rng(n)
    finite = np.array([c for c in range(256) if c & 0x7F != 0x7F], dtype=np.uint8)
    codes = finite[rng.integers(0, finite.size, size=n)]
    s = rng.random(3, dtype=np.float32)
    want_enc, want_adj, want_rounded = ref.reencode_e4m3fn_half(codes, s)
    enc, adj, rounded = gk.reencode_e4m3fn_half(_fp8(codes), torch.from_numpy(s).cuda())
    assert np.array_equal(_u8(enc), want_enc) and rounded == want_rounded
    assert np.array_equal(adj.cpu().numpy(), want_adj)
    # unaligned views take the byte path
    if n > 3:
        base = _fp8(np.concatenate([np.zeros(1, np.uint8), codes]))
        enc2, _, r2 = gk.reencode_e4m3fn_half(base[1:], torch.from_numpy(s).cuda())
        assert np.array_equal(_u8(enc2), want_enc) and r2 == want_rounded


def _cfg2_tensor(rows, cols, seed=0):
    # N(0, 0.02) with 0.1 % of entries scaled by 50 (sign kept)
    g = torch.Generator().manual_seed(seed)
    t = torch.randn((rows, cols), generator=g) * 0.02
    mask = torch.rand((rows, cols), generator=g) < 1e-3
    return torch.where(mask, t * 50, t).contiguous()


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (300, 200), (129, 130), (1, 1), (8, 1027)])
@pytest.mark.parametrize("half", [False, True])
def test_quantize_block128_matches_oracle(gk, shape, half):
    t = _cfg2_tensor(*shape, seed=shape[0] + shape[1])
    t[0, 0] = 0.0
    if shape[0] > 140:
        t[128:256, :128] = 0.0                                     # an all-zero tile: amax floor 1e-10
    want_codes, want_scales = ref.quantize_block128(t.numpy(), native_half=half)
    codes, scales = gk.quantize_block128(t.cuda(), native_half=half)
    assert np.array_equal(scales.cpu().numpy(), want_scales)
    assert np.array_equal(_u8(codes), want_codes)


def test_quantize_block128_rounding_ties(gk):
    # values placed exactly half-way between E4M3 grid points, and tiny values around the amax floor
    grid = ref.e4m3_values()[:127].astype(np.float64)
    mids = ((grid[:-1] + grid[1:]) / 2).astype(np.float32)
    t = np.zeros((128, 128), dtype=np.float32)
    t.reshape(-1)[:126] = mids
    t.reshape(-1)[126:252] = -mids
    t[127, 127] = 448.0                                              # scale becomes exactly ~1
    for arr in (t, t * np.float32(1e-12), t * np.float32(3e-13)):
        for half in (False, True):
            want_codes, want_scales = ref.quantize_block128(arr, native_half=half)
            codes, scales = gk.quantize_block128(torch.from_numpy(arr).cuda(), native_half=half)
            assert np.array_equal(scales.cpu().numpy(), want_scales)
            assert np.array_equal(_u8(codes), want_codes)


def test_quantize_block128_full_config(gk):
    # the codec configuration: fp32 [8192, 8192], N(0, 0.02) with 0.1 % outliers at 50x
    t = _cfg2_tensor(8192, 8192)
    want_codes, want_scales = ref.quantize_block128(t.numpy(), native_half=True)
    codes, scales = gk.quantize_block128(t.cuda(), native_half=True)
    assert np.array_equal(scales.cpu().numpy(), want_scales)
    assert np.array_equal(_u8(codes), want_codes)
    # two-step path (OCP quantize, then re-encode) gives the same bytes and counts roundings
    ocp, s1 = gk.quantize_block128(t.cuda())
    enc, s2, rounded = gk.reencode_e4m3fn_half(ocp, s1)
    assert torch.equal(enc.view(torch.uint8), codes.view(torch.uint8)) and torch.equal(s2, scales)
    w_enc, _, w_rounded = ref.reencode_e4m3fn_half(_u8(ocp), s1.cpu().numpy())
    assert rounded == w_rounded and np.array_equal(_u8(enc), w_enc)
    # decode round trip: every element within half an E4M3 step of the block's grid
    back = gk.decode_e4m3(codes, scales)
    want_back = ref.decode_block128(want_codes, want_scales)
    assert np.array_equal(back.cpu().numpy(), want_back)
    err = (back.cpu() - t).abs()
    bound = scales.cpu().repeat_interleave(128, 0).repeat_interleave(128, 1) * 16.0   # half-range step at the top binade
    assert bool((err <= bound).all())


@pytest.mark.parametrize("shape", [(1, 128), (37, 384), (5, 200), (3, 1000), (64, 4096), (256, 1024), (7, 130)])
@pytest.mark.parametrize("half", [False, True])
def test_quantize_act_matches_oracle(gk, shape, half):
    g = torch.Generator().manual_seed(shape[0] * 7 + shape[1])
    x = torch.randn(shape, generator=g)
    if shape[0] > 2:
        x[1] = 0.0                                                 # all-zero row
        x[0, :128] = 0.0                                           # all-zero group
        x[2] *= 1e-13                                              # below the 1e-10 amax floor
    x = x.to(torch.bfloat16)
    want_codes, want_scales = ref.quantize_act_1x128(x.float().numpy(), native_half=half)
    codes, scales = gk.quantize_act_1x128(x.cuda(), native_half=half)
    assert tuple(scales.shape) == want_scales.shape
    assert np.array_equal(scales.cpu().numpy(), want_scales)
    assert np.array_equal(_u8(codes), want_codes)


def test_quantize_act_flags_nonfinite(gk):
    x = torch.randn((4, 256)).to(torch.bfloat16)
    gk.quantize_act_1x128(x.cuda(), check_finite=True)
    for bad in (float("inf"), float("nan")):
        y = x.clone()
        y[3, 200] = bad
        with pytest.raises(ValueError):
            gk.quantize_act_1x128(y.cuda(), check_finite=True)


@pytest.mark.parametrize("shape", [(2, 128), (256, 384), (130, 136), (5, 7)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_matches_oracle(gk, shape, dtype):
    rng = np.random.default_rng(shape[0] * 13 + shape[1])
    finite = np.array([c for c in range(256) if c & 0x7F != 0x7F], dtype=np.uint8)
    codes = np.ascontiguousarray(finite[rng.integers(0, finite.size, size=shape)])
    scales = rng.random(((shape[0] + 127) // 128, (shape[1] + 127) // 128), dtype=np.float32) * np.float32(0.01)
    want = ref.decode_block128(codes, scales, out_bf16=dtype == torch.bfloat16)
    got = gk.decode_e4m3(_fp8(codes), torch.from_numpy(scales).cuda(), out_dtype=dtype)
    assert got.dtype == dtype
    assert np.array_equal(got.float().cpu().numpy(), want)


def test_decode_all_codes(gk):
    codes = np.arange(256, dtype=np.uint8).reshape(2, 128)
    got = gk.decode_e4m3(_fp8(codes), torch.ones((1, 1), device="cuda")).cpu().numpy().reshape(-1)
    want = ref.e4m3_values()
    ok = np.isfinite(want)
    assert np.array_equal(got[ok], want[ok]) and np.isnan(got[~ok]).all()


@pytest.mark.parametrize("n", [1, 15, 4096 + 3, (1 << 20) + 17])
def test_reencode_in_place_through_the_c_abi(gk, n):
    """codes_out == codes_in and scales_out == scales_in, which the header allows: same bytes as out of place."""
    from gaudi_kernels_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(n)
    codes = rng.integers(0, 256, size=n, dtype=np.uint8)
    codes[(codes & 0x7f) == 0x7f] ^= 0x01
    scales = rng.random(7, dtype=np.float32)
    want_codes, want_scales, want_rounded = ref.reencode_e4m3fn_half(codes, scales)
    holder = torch.zeros(n + 32, dtype=torch.uint8, device="cuda")
    for offset in (0, 5):                                            # aligned and unaligned start
        buf = holder[offset:offset + n]
        buf.copy_(torch.from_numpy(codes))
        sc = torch.from_numpy(scales).cuda()
        st = torch.zeros(4, dtype=torch.int32, device="cuda")
        rc = lib.bfp8_reencode_half(buf.data_ptr(), buf.data_ptr(), n, sc.data_ptr(), sc.data_ptr(), sc.numel(),
                                    st.data_ptr(), st.data_ptr() + 8, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        host = st.cpu()
        assert int(host[2]) == 0 and (int(host[1]) << 32 | (int(host[0]) & 0xFFFFFFFF)) == want_rounded
        assert np.array_equal(buf.cpu().numpy(), want_codes)
        assert np.array_equal(sc.cpu().numpy(), want_scales)
