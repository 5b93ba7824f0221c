"""B200-native block-FP8 path of gaudi-kernels: E4M3 codec, block-amax quantizers, block-scaled GEMM.

The public names follow the reference package (`reencode_e4m3fn_half`, `reference`); all compute runs
in libbfp8.so (hand-written sm_100a CUDA behind a C ABI).  PyTorch supplies tensors and streams only.
"""

from .block_fp8_gemm import (gemm_block_fp8, gemm_block_fp8_swiglu, gemm_token_channel_fp8, prepare_weight,
                             prepare_weight_swiglu, reference, set_weights_at_rest, silu_and_mul)
from .fp8_codec import (decode_e4m3, quantize_act_1x128, quantize_act_token, quantize_block128,
                        reencode_e4m3fn_half, silu_quantize_act_1x128)

__all__ = ["reencode_e4m3fn_half", "reference", "gemm_block_fp8", "prepare_weight",
           "quantize_block128", "quantize_act_1x128", "decode_e4m3", "quantize_act_token", "gemm_token_channel_fp8",
           "prepare_weight_swiglu", "gemm_block_fp8_swiglu", "silu_and_mul", "silu_quantize_act_1x128",
           "set_weights_at_rest"]
