"""The CPU oracle against the reference's own vectors and against fixtures the reference produced."""

import numpy as np
import pytest
import torch

import cases
from oracle import block_fp8_ref, fp8_codec_ref


def _value(mag):
    e, f = divmod(mag, 8)
    return f * 2.0 ** -9 if e == 0 else (1.0 + f / 8.0) * 2.0 ** (e - 7)


def test_codec_all_finite_codes_nearest_even():
    # the exhaustive vector of the reference's tests/test_fp8_codec.py:16-42
    src = np.array([c for c in range(256) if c & 0x7F != 0x7F], dtype=np.uint8)
    scales = np.array([0.0, 0.25, 1.0e30], dtype=np.float32)
    enc, adj, rounded = fp8_codec_ref.reencode_e4m3fn_half(src, scales)
    expected, inexact = [], 0
    for c in src.tolist():
        want = _value(c & 0x7F) / 2.0
        dist = [abs(_value(k) - want) for k in range(0x78)]
        best = min(dist)
        ties = [k for k, d in enumerate(dist) if d == best]
        sel = next(k for k in ties if k % 2 == 0) if len(ties) > 1 else ties[0]
        expected.append((c & 0x80) | sel)
        inexact += best != 0
    assert enc.tolist() == expected
    assert np.array_equal(adj, scales * 2)
    assert rounded == inexact == 16
    assert enc[src.tolist().index(0x01)] == 0x00 and enc[src.tolist().index(0x81)] == 0x80


def test_codec_known_answer_and_errors():
    # tests/test_fp8_codec.py:44-68
    w = np.array([[0x08, 0x10, 0x78], [0x03, 0x7E, 0x80]], dtype=np.uint8)
    enc, adj, rounded = fp8_codec_ref.reencode_e4m3fn_half(w, np.array([[0.25, 0.5]], dtype=np.float32))
    assert enc.tolist() == [[4, 8, 112], [2, 118, 128]] and rounded == 1
    assert adj.tolist() == [[0.5, 1.0]]
    one = np.ones(1, dtype=np.float32)
    for code in (0x7F, 0xFF):
        with pytest.raises(ValueError, match="nonfinite"):
            fp8_codec_ref.reencode_e4m3fn_half(np.array([0, code], dtype=np.uint8), one)
    z = np.zeros(2, dtype=np.uint8)
    for bad in (float("nan"), float("inf"), -1.0, np.finfo(np.float32).max):
        with pytest.raises(ValueError):
            fp8_codec_ref.reencode_e4m3fn_half(z, np.array([bad], dtype=np.float32))
    with pytest.raises(ValueError):
        fp8_codec_ref.reencode_e4m3fn_half(w.T, one)
    with pytest.raises(ValueError):
        fp8_codec_ref.reencode_e4m3fn_half(w, one.astype(np.float64))


def test_codec_matches_reference_fixtures(golden_codec):
    for name, (codes, scales) in cases.codec_cases().items():
        assert np.array_equal(codes, golden_codec[name + ".codes"])
        enc, adj, rounded = fp8_codec_ref.reencode_e4m3fn_half(codes, scales)
        assert np.array_equal(enc, golden_codec[name + ".encoded"]), name
        assert np.array_equal(adj, golden_codec[name + ".adjusted"]), name
        assert rounded == int(golden_codec[name + ".rounded"]), name


def test_half_table_equals_two_step_cast():
    # block_fp8_oracle.py:32-33 "(q*.5).to(float8_e4m3fn)" is the codec's byte map
    finite = torch.tensor([c for c in range(256) if c & 0x7F != 0x7F], dtype=torch.uint8)
    halved = (finite.view(torch.float8_e4m3fn).float() * .5).to(torch.float8_e4m3fn).view(torch.uint8)
    assert np.array_equal(halved.numpy(), fp8_codec_ref.half_table()[finite.numpy()])


def test_decode_table_matches_torch():
    vals = fp8_codec_ref.e4m3_values()
    tv = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    ok = np.isfinite(tv)
    assert ok.sum() == 254 and np.array_equal(vals[ok], tv[ok]) and np.isnan(vals[~ok]).all()


def test_rne_cast_torch_equals_grid_search():
    rng = np.random.default_rng(5)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * 100,
        rng.standard_normal(200000).astype(np.float32) * 0.01,
        (np.arange(-1024, 1025, dtype=np.float32) * np.float32(2.0 ** -10)),   # ties on the 2^-9 grid
        np.array([448.0, -448.0, 447.9, 464.0, 0.0, -0.0, 2.0 ** -10, -(2.0 ** -10), 3 * 2.0 ** -10], np.float32),
    ])
    x = np.clip(x, -448, 448).astype(np.float32)
    assert np.array_equal(fp8_codec_ref.cast_e4m3fn_rne(x), fp8_codec_ref.cast_e4m3fn_rne_search(x))


def test_gemm_oracle_matches_reference_fixtures(golden_gemm, gemm_cases):
    for name, c in gemm_cases.items():
        assert cases.digest(c) == golden_gemm[name + ".input_digest"].tobytes(), name
        x = torch.from_numpy(c["x_bf16_bits"]).view(torch.bfloat16)
        w = torch.from_numpy(c["w_codes"]).view(torch.float8_e4m3fn)
        s = torch.from_numpy(c["w_scales"])
        b = None if c["bias"] is None else torch.from_numpy(c["bias"])
        for half in (False, True):
            y64, y = block_fp8_ref.reference_rows(x, w, s, native_half=half, bias=b)
            want = golden_gemm[f"{name}.y_bits.half{int(half)}"]
            assert np.array_equal(y.view(torch.int16).numpy(), want), (name, half)
            assert torch.equal(y64.to(torch.bfloat16), y)


def test_gemm_oracle_chunking_is_row_independent(gemm_cases):
    c = gemm_cases["sim_edges"]
    x = torch.from_numpy(c["x_bf16_bits"]).view(torch.bfloat16)
    w = torch.from_numpy(c["w_codes"]).view(torch.float8_e4m3fn)
    s = torch.from_numpy(c["w_scales"])
    full = block_fp8_ref.reference_rows(x, w, s, native_half=True)[0]
    by7 = block_fp8_ref.reference_rows(x, w, s, native_half=True, chunk_rows=7)[0]
    assert torch.equal(full, by7)


def test_quantizers_match_oracle_lines(gemm_cases):
    # the numpy 1x128 quantizer equals the torch lines used inside the GEMM oracle
    c = gemm_cases["sim_edges"]
    x = torch.from_numpy(c["x_bf16_bits"]).view(torch.bfloat16)
    for half in (False, True):
        qa, sa = block_fp8_ref.quantize_rows(x, 3, half)
        codes, scales = fp8_codec_ref.quantize_act_1x128(x.float().numpy(), native_half=half)
        assert np.array_equal(fp8_codec_ref.e4m3_values()[codes].reshape(37, 3, 128), qa.numpy())
        assert np.array_equal(scales, sa.numpy().reshape(37, 3))


def test_reference_gate_row_l2(gemm_cases):
    # the reference's device gate (tests/fp8_hybrid_tpcsim_test.cpp:353-379) holds for the oracle itself
    c = gemm_cases["sim_edges"]
    x = torch.from_numpy(c["x_bf16_bits"]).view(torch.bfloat16)
    w = torch.from_numpy(c["w_codes"]).view(torch.float8_e4m3fn)
    s = torch.from_numpy(c["w_scales"])
    b = torch.from_numpy(c["bias"])
    y = block_fp8_ref.reference(x, w, s, native_half=True, bias=b).double()
    r = block_fp8_ref.w8a8_fp64_reference(x, w, s, bias=b).double()
    num = ((y - r) ** 2).sum(1).sqrt()
    den = (r ** 2).sum(1).sqrt()
    assert bool(((num / den.clamp_min(1e-300)) <= 0.01).all())
