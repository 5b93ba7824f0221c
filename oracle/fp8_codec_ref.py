"""CPU restatement of the OCP -> Gaudi2 half-range E4M3 codec. TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA codec kernels: only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may import it.  The shipped
package never does.

Follows python/gaudi_kernels/fp8_codec.py:14-53 of tracycam/gaudi-kernels (the
byte map at :36-40, the rejection of 0x7f/0xff at :48-49, the rounded-element
count at :50, the scale doubling and overflow check at :30-32).  Parity is pinned
by the reference's own vectors in tests/test_fp8_codec.py (exhaustive 254-code
map :16-42, known answer :56-64, error cases :44-54, :65-68) and by fixtures
generated from the reference itself (tests/golden/).

The decode helper follows the value() function of tests/test_fp8_codec.py:8-12.
The block-amax quantizers restate python/gaudi_kernels/block_fp8_oracle.py:27-28
(and :31-35 for the half-range step); the reference has no 128x128 weight
quantizer of its own, so that function's parity is unpinned beyond the 1x128 rule
it reuses.
"""

import numpy as np
import torch

BLOCK = 128
E4M3_MAX = 448.0
INV_448_F32 = np.float32(1.0 / 448.0)   # block_fp8_oracle.py:27  "* (1.0 / 448.0)" in fp32
AMAX_FLOOR_F32 = np.float32(1e-10)      # block_fp8_oracle.py:27  clamp_min(1e-10)


def half_table():
    """256-entry byte map: OCP E4M3FN code -> Gaudi2 code of half the value, RNE.

    fp8_codec.py:36-40.  Normal codes (magnitude >= 16) lose one exponent step
    (magnitude - 8); the low end shifts the significand right with
    round-to-nearest-even: odd magnitudes round up only when the result would
    otherwise be odd.
    """
    c = np.arange(256, dtype=np.uint16)
    mag = c & 0x7F
    lo = (mag >> 1) + ((mag & 1) & ((mag >> 1) & 1))
    half = np.where(mag >= 16, mag - 8, lo)
    return ((c & 0x80) | half).astype(np.uint8)


def reencode_e4m3fn_half(weight_u8, scales_f32):
    """numpy restatement of fp8_codec.py:14-53 on raw bytes.

    weight_u8: uint8 array of OCP E4M3FN codes (any shape, non-empty, C-contiguous).
    scales_f32: float32 array, finite, non-negative, doubling must stay finite.
    Returns (encoded uint8 same shape, float32 scales*2, int rounded).
    Raises ValueError like the reference ("nonfinite" for 0x7f / 0xff codes).
    """
    w = np.asarray(weight_u8)
    s = np.asarray(scales_f32)
    if w.dtype != np.uint8 or w.size == 0 or not w.flags.c_contiguous:
        raise ValueError("expected a nonempty contiguous E4M3FN weight")
    if (s.dtype != np.float32 or s.size == 0 or not s.flags.c_contiguous
            or not np.all(np.isfinite(s)) or np.any(s < 0)):
        raise ValueError("expected nonempty contiguous finite nonnegative FP32 scales")
    with np.errstate(over="ignore"):
        doubled = (s * np.float32(2.0)).astype(np.float32)
    if not np.all(np.isfinite(doubled)):
        raise ValueError("doubling FP8 scales overflows FP32")
    mag = w & 0x7F
    if np.any(mag == 0x7F):
        raise ValueError("nonfinite OCP E4M3FN checkpoint code")
    rounded = int(np.count_nonzero((mag < 16) & ((mag & 1) != 0)))
    return half_table()[w], doubled, rounded


def e4m3_values():
    """float32 value of each of the 256 OCP E4M3FN codes (0x7f / 0xff -> NaN).

    tests/test_fp8_codec.py:8-12: exponent field 0 is the 2^-9 subnormal grid,
    otherwise (1 + m/8) * 2^(e-7).  Codes up to magnitude 0x77 mean the same in
    the Gaudi2 encoding, and re-encoded weights never exceed 0x76.
    """
    out = np.empty(256, dtype=np.float32)
    for c in range(256):
        m = c & 0x7F
        e, f = divmod(m, 8)
        v = f * 2.0 ** -9 if e == 0 else (1.0 + f / 8.0) * 2.0 ** (e - 7)
        if m == 0x7F:
            v = float("nan")
        out[c] = -v if c & 0x80 else v
    return out


def cast_e4m3fn_rne_search(x_f32):
    """fp32 -> OCP E4M3FN code, round-to-nearest-even, by searching the value grid.

    Independent of torch's cast (used to cross-check it).  Inputs must already be
    clamped to [-448, 448].  Sign of zero and of values that round to zero is kept.
    """
    x = np.asarray(x_f32, dtype=np.float32)
    grid = e4m3_values()[:127].astype(np.float64)          # magnitudes 0 .. 448
    a = np.abs(x).astype(np.float64)
    hi = np.searchsorted(grid, a, side="left")
    hi = np.minimum(hi, 126)
    lo = np.maximum(hi - 1, 0)
    d_lo = a - grid[lo]
    d_hi = grid[hi] - a
    take_lo = (d_lo < d_hi) | ((d_lo == d_hi) & ((lo & 1) == 0))
    code = np.where(take_lo, lo, hi).astype(np.uint8)
    return code | (np.signbit(x).astype(np.uint8) << 7)


def cast_e4m3fn_rne(x_f32):
    """fp32 -> OCP E4M3FN code through torch's CPU cast, as block_fp8_oracle.py:28 does."""
    t = torch.from_numpy(np.ascontiguousarray(x_f32, dtype=np.float32))
    return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def _scale_from_amax(amax_f32):
    # block_fp8_oracle.py:27: clamp_min(1e-10) then one fp32 multiply by fp32(1/448).
    return (np.maximum(amax_f32.astype(np.float32), AMAX_FLOOR_F32) * INV_448_F32).astype(np.float32)


def _quantize(a_f32, sa_f32):
    # block_fp8_oracle.py:28: IEEE fp32 division, clamp to +-448, RNE cast.
    q = (a_f32 / sa_f32).astype(np.float32)
    q = np.clip(q, np.float32(-E4M3_MAX), np.float32(E4M3_MAX))
    return cast_e4m3fn_rne(q)


def quantize_act_1x128(x_f32, native_half=False):
    """1x128 activation quantizer, block_fp8_oracle.py:25-28 (+ :31-35 when native_half).

    x_f32: float32 [M, K] holding bf16-representable values.  K is zero-padded to
    a multiple of 128 for the amax but codes are returned for the K real columns.
    Returns (codes uint8 [M, K], scales float32 [M, G]).
    """
    x = np.asarray(x_f32, dtype=np.float32)
    m, k = x.shape
    g = (k + BLOCK - 1) // BLOCK
    a = np.zeros((m, g * BLOCK), dtype=np.float32)
    a[:, :k] = x
    a = a.reshape(m, g, BLOCK)
    sa = _scale_from_amax(np.abs(a).max(axis=-1, keepdims=True))
    codes = _quantize(a, sa).reshape(m, g * BLOCK)[:, :k]
    sa = sa.reshape(m, g)
    if native_half:
        codes = half_table()[codes]
        sa = (sa * np.float32(2.0)).astype(np.float32)
    return np.ascontiguousarray(codes), np.ascontiguousarray(sa)


def quantize_block128(w_f32, native_half=False):
    """128x128 block-amax weight quantizer (new API; the 1x128 rule over a square tile).

    w_f32: float32 [R, C].  Ragged edges are zero-padded for the amax.
    Returns (codes uint8 [R, C] in OCP E4M3FN (or half-range if native_half),
             scales float32 [ceil(R/128), ceil(C/128)] (doubled if native_half)).
    """
    w = np.asarray(w_f32, dtype=np.float32)
    r, c = w.shape
    rb, cb = (r + BLOCK - 1) // BLOCK, (c + BLOCK - 1) // BLOCK
    p = np.zeros((rb * BLOCK, cb * BLOCK), dtype=np.float32)
    p[:r, :c] = w
    t = p.reshape(rb, BLOCK, cb, BLOCK)
    s = _scale_from_amax(np.abs(t).max(axis=(1, 3)))
    codes = _quantize(t, s[:, None, :, None]).reshape(rb * BLOCK, cb * BLOCK)[:r, :c]
    if native_half:
        codes = half_table()[codes]
        s = (s * np.float32(2.0)).astype(np.float32)
    return np.ascontiguousarray(codes), np.ascontiguousarray(s)


def decode_block128(codes_u8, scales_f32, out_bf16=False):
    """value(code) * block scale in fp32 (one multiply), optionally rounded to bf16 (RNE).

    codes_u8: uint8 [R, C]; scales_f32: [ceil(R/128), ceil(C/128)].
    Returns float32 [R, C] (bf16-rounded values when out_bf16).
    """
    codes = np.asarray(codes_u8, dtype=np.uint8)
    r, c = codes.shape
    s = np.asarray(scales_f32, dtype=np.float32)
    s_full = np.repeat(np.repeat(s, BLOCK, axis=0)[:r], BLOCK, axis=1)[:, :c]
    out = (e4m3_values()[codes] * s_full).astype(np.float32)
    if out_bf16:
        out = torch.from_numpy(out).to(torch.bfloat16).float().numpy()
    return out
