"""Seeded input builders shared by make_golden.py and the test-suite.

Inputs come from numpy's PCG64 generator (bit-reproducible across machines), not
from any dataset.  Shapes follow the block-FP8 path's configurations: the
M=256, K=N=1024 CPU case, a biased ragged-M case, a case whose K and N are not
multiples of 128, and cases that re-state the input recipe of the reference's
simulator test (tests/fp8_hybrid_tpcsim_test.cpp:187-231 of tracycam/gaudi-kernels:
one all-zero row, one all-zero group, 12x / 1.5x envelopes, structured weight
codes 8..125, the (0.5 + 0.25*((5nb+3g)%11))*1e-3 scale grid, and the
1e-15 / 1e-12 "tiny" envelopes) at that test's five shapes (:388-392): (37, 256, 384)
with bias, (4, 128, 256) tiny, and the long-K ones (4, 256, 7168), a 28-group case
(the reference runs K=7168 a second time in chunks of 28 groups; a contraction that
is not chunked has no such mode, so the case is K = 28 groups), and (2, 128, 22016).
The long-K cases also follow the test's sign rule for odd groups (:213-218): the
weight sign follows whether row 0's activations of the two neighbouring groups agree
in sign, which makes consecutive K blocks add up instead of cancelling.
"""

import hashlib
import os
import sys

import numpy as np
import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from oracle import fp8_codec_ref as codec_ref  # noqa: E402


def to_bf16_bits(a_f32):
    t = torch.from_numpy(np.ascontiguousarray(a_f32, dtype=np.float32)).to(torch.bfloat16)
    return t.view(torch.int16).numpy().copy()


def bf16_bits_to_f32(bits):
    return torch.from_numpy(np.ascontiguousarray(bits)).view(torch.bfloat16).float().numpy()


def digest(case):
    h = hashlib.sha256()
    for key in ("x_bf16_bits", "w_codes", "w_scales", "bias"):
        v = case[key]
        if v is not None:
            h.update(np.ascontiguousarray(v).tobytes())
    return h.digest()


def _gaussian_case(seed, m, k, n, with_bias, store_inputs):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    codes, scales = codec_ref.quantize_block128(w)
    bias = None
    if with_bias:
        bias = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    return dict(x_bf16_bits=to_bf16_bits(x), w_codes=codes, w_scales=scales, bias=bias,
                store_inputs=store_inputs)


def _simulator_style_case(seed, m, n, k, with_bias, tiny, correlated_signs=False, store_inputs=True):
    rng = np.random.default_rng(seed)
    groups, blocks = k // 128, n // 128
    x = np.zeros((m, k), dtype=np.float32)
    for r in range(m):
        if not tiny and r == 1:
            continue                                   # an entire all-zero row
        for g in range(groups):
            if not tiny and r == 0 and g == 0:
                continue                               # an all-zero group
            if tiny:
                env = 1.0e-15 if g & 1 else 1.0e-12
            else:
                env = 12.0 if (g // 2) % 4 == 0 else 1.5
            x[r, g * 128:(g + 1) * 128] = rng.standard_normal(128, dtype=np.float32) * np.float32(env)
    col = np.arange(n)[:, None, None]
    g = np.arange(groups)[None, :, None]
    i = np.arange(128)[None, None, :]
    codes = ((col * 17 + g * 31 + i * 7) % 118 + 8).astype(np.uint8)
    sign = np.broadcast_to(((col * 3 + g * 5 + i) & 1).astype(np.uint8), (n, groups, 128)).copy()
    if correlated_signs:
        # odd groups, lanes not divisible by 5: sign set where row 0's bf16 activations at (g - 1, i) and (g, i)
        # have the same sign (zero counts as non-negative)
        x0 = bf16_bits_to_f32(to_bf16_bits(x[0])).reshape(groups, 128)
        neg = x0 < 0
        same = np.zeros((groups, 128), dtype=np.uint8)
        same[1:] = (neg[1:] == neg[:-1]).astype(np.uint8)
        rule = ((np.arange(groups)[:, None] & 1) == 1) & ((np.arange(128)[None, :] % 5) != 0)
        sign = np.where(rule[None], same[None], sign).astype(np.uint8)
    codes = (codes | (sign << 7)).reshape(n, k)
    nb = np.arange(blocks)[:, None]
    gg = np.arange(groups)[None, :]
    scales = ((0.5 + 0.25 * ((nb * 5 + gg * 3) % 11)) * 1e-3).astype(np.float32)
    bias = None
    if with_bias:
        c = np.arange(n)
        bias = (np.where(c & 1, -0.125, 0.125) + c * 1e-4).astype(np.float32)
    return dict(x_bf16_bits=to_bf16_bits(x), w_codes=np.ascontiguousarray(codes),
                w_scales=np.ascontiguousarray(scales), bias=bias, store_inputs=store_inputs)


def gemm_cases():
    return {
        "cfg1": _gaussian_case(0, 256, 1024, 1024, False, False),
        "small_bias": _gaussian_case(1, 5, 384, 256, True, True),
        "ragged": _gaussian_case(2, 3, 208, 136, True, True),
        "sim_edges": _simulator_style_case(3, 37, 256, 384, True, False),
        "sim_tiny": _simulator_style_case(4, 4, 128, 256, False, True),
        "sim_k7168": _simulator_style_case(5, 4, 256, 7168, False, False, True, False),
        "sim_k3584": _simulator_style_case(6, 4, 256, 3584, False, False, True, False),
        "sim_k22016": _simulator_style_case(7, 2, 128, 22016, False, False, True, False),
    }


def codec_cases():
    rng = np.random.default_rng(7)
    finite = np.array([c for c in range(256) if c & 0x7F != 0x7F], dtype=np.uint8)
    rand = finite[rng.integers(0, finite.size, size=(257, 513))]
    return {
        "all_finite": (finite, np.array([0.0, 0.25, 1.0e30], dtype=np.float32)),
        "known": (np.array([[0x08, 0x10, 0x78], [0x03, 0x7E, 0x80]], dtype=np.uint8),
                  np.array([[0.25, 0.5]], dtype=np.float32)),
        "random": (np.ascontiguousarray(rand),
                   rng.random((3, 5), dtype=np.float32) * np.float32(0.01)),
    }
