"""CPU restatement of the reference's SwiGLU step (silu_and_mul) after the gate/up GEMM. TEST INFRASTRUCTURE ONLY.

Only the test-suite imports this module.  The reference implements the step as the Gaudi2 TPC kernel
gk_silu_and_mul_bf16_v1 and ships no CPU definition or test vector for it (tests/generic_dense_guids_test.cpp:38
only checks that the kernel is registered), so parity is unpinned: this file restates the kernel's arithmetic
from its source:

* silu_and_mul_bf16 - csrc/tpc/generic_dense/silu_and_mul_bf16.c:4-13 and :16-75: the input is bf16
  [rows, 2 * width], gate in columns [0, width) and up in columns [width, 2 * width) (:29); both are widened
  to fp32, silu(g) = g / (1 + exp(-g)) with a refined quotient (:5-9), exactly 0 for g <= -88 (:10), NaN passed
  through (:11-12); the product with up is rounded to bf16 once, round-to-nearest-even (:15, :59-60).
  Evaluated in FP64 here and rounded to fp32 before the product, which is what a correctly rounded fp32
  quotient gives; the TPC's exp and reciprocal approximations can differ from it in the last fp32 bits, far
  below the bf16 rounding of the result.
* interleave_gate_up - the row order bfp8_swiglu_interleave_weight produces (no reference counterpart: the
  reference's GEMM output is simply read at `col` and `col + width`).
"""

import numpy as np
import torch


def silu_and_mul_bf16(gate_up):
    """gate_up: torch bf16 [rows, 2 * width] -> torch bf16 [rows, width]."""
    if gate_up.dtype != torch.bfloat16 or gate_up.ndim != 2 or gate_up.shape[1] % 2:
        raise ValueError("bf16 [rows, 2 * width] expected")
    width = gate_up.shape[1] // 2
    g = gate_up[:, :width].double()
    u = gate_up[:, width:].float()
    s = (g / (1.0 + torch.exp(-g))).float()
    s = torch.where(g <= -88.0, torch.zeros_like(s), s)
    s = torch.where(torch.isnan(g), g.float(), s)
    return (s * u).to(torch.bfloat16)


def interleave_gate_up(w, chunk=64):
    """numpy [2 * I, K] (gate rows then up rows) -> rows interleaved in chunks of `chunk` outputs."""
    w = np.asarray(w)
    inter = w.shape[0] // 2
    if w.shape[0] % 2 or inter % chunk:
        raise ValueError("2 * I rows with I a multiple of the chunk expected")
    gate = w[:inter].reshape(inter // chunk, chunk, -1)
    up = w[inter:].reshape(inter // chunk, chunk, -1)
    return np.ascontiguousarray(np.stack([gate, up], axis=1).reshape(w.shape[0], -1))
