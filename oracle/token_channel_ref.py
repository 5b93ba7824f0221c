"""CPU restatement of the reference's per-token / per-channel FP8 variant. TEST INFRASTRUCTURE ONLY.

Only the test-suite imports this module.  The reference realises this variant as Gaudi2 TPC kernels
around an MME GEMM and ships no CPU definition or test vector for it, so parity is unpinned: this file
restates the kernels' arithmetic from their sources:

* quantize_act_token - csrc/tpc/block_fp8_framework/activation_token.c:4-26 with the helpers of
  activation_quant_common.h:3-30: amax over the row, 1 substituted for an all-zero row (:17), the
  FMA-corrected scale (activation_quant_common.h:3-7) which is the correctly rounded amax / 448, the
  FMA-corrected quotient x / scale (:9-12), clamp to 448, round-to-nearest-even to OCP E4M3 with the 2^-9
  subnormal grid (:13-19), halving with RNE (:20,23-30), stored scale * 2 (activation_token.c:24).
* gemm_token_channel - the FP32 accumulation of the quantized operands followed by
  csrc/tpc/block_fp8_framework/channel_finish.c:2-18: (partial * act) * w_scale + bias, bf16 RNE.
  Evaluated in FP64 here; products of E4M3 values are exact in FP64.
"""

import numpy as np
import torch

from . import fp8_codec_ref as codec


def quantize_act_token(x_f32, native_half=True):
    x = np.asarray(x_f32, dtype=np.float32)
    amax = np.abs(x).max(axis=1, keepdims=True).astype(np.float32)
    amax = np.where(amax == 0, np.float32(1.0), amax).astype(np.float32)
    scale = (amax / np.float32(448.0)).astype(np.float32)
    q = np.clip((x / scale).astype(np.float32), np.float32(-448.0), np.float32(448.0))
    codes = codec.cast_e4m3fn_rne(q)
    scale = scale.reshape(-1)
    if native_half:
        codes = codec.half_table()[codes]
        scale = (scale * np.float32(2.0)).astype(np.float32)
    return np.ascontiguousarray(codes), np.ascontiguousarray(scale)


def gemm_token_channel(a_codes, a_scales, w_codes, w_scales, bias=None):
    """Returns (y_fp64 [M, N], y_bf16 [M, N])."""
    vals = torch.from_numpy(codec.e4m3_values().astype(np.float64))
    a = vals[torch.from_numpy(np.asarray(a_codes)).long()]
    w = vals[torch.from_numpy(np.asarray(w_codes)).long()]
    y = (a @ w.T) * torch.from_numpy(np.asarray(a_scales, dtype=np.float32)).double().view(-1, 1)
    y = y * torch.from_numpy(np.asarray(w_scales, dtype=np.float32)).double().view(1, -1)
    if bias is not None:
        y = y + torch.from_numpy(np.asarray(bias, dtype=np.float32)).double().view(1, -1)
    return y, y.to(torch.bfloat16)
