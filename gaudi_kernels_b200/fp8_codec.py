"""E4M3 codec and block-amax quantizers on B200, behind the reference's function signatures.

`reencode_e4m3fn_half(weight, scales)` is a drop-in for
python/gaudi_kernels/fp8_codec.py:14-53 of tracycam/gaudi-kernels: same arguments, same
(encoded, doubled scales, rounded count) result, same ValueError behaviour ("nonfinite" for
0x7f / 0xff codes; bad dtype, layout or scales rejected; inputs never modified).  The work is done
by the CUDA kernels of libbfp8.so; there is no CPU implementation in this package.

Tensors may live on a CUDA device (results stay there) or on the host (they are copied to the
current CUDA device, processed, and the results copied back - the call a CPU user of the
reference would make).

The quantizers and the decoder are siblings in the same style; the reference has the 1x128
activation rule inline in block_fp8_oracle.py:25-28 and no weight quantizer or decoder at all.
"""

import torch

from . import _lib

BLOCK = 128


def _device_for(*tensors):
    for t in tensors:
        if t.device.type == "cuda":
            return t.device
    if not torch.cuda.is_available():
        raise _lib.Bfp8Error("a CUDA device is required; this package has no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def _stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def _status_buffer(device):
    # [0:2] 64-bit rounded counter, [2] status word, [3] padding
    return torch.zeros(4, dtype=torch.int32, device=device)


def _read_status(buf):
    host = buf.cpu()                       # synchronises with the launching stream
    lo, hi, status = int(host[0]) & 0xFFFFFFFF, int(host[1]) & 0xFFFFFFFF, int(host[2]) & 0xFFFFFFFF
    return (hi << 32) | lo, status


def reencode_e4m3fn_half(weight, scales):
    """Return (encoded bytes, doubled FP32 scales, rounded element count).

    Mirrors fp8_codec.py:14-53: `weight` is a non-empty contiguous float8_e4m3fn tensor of OCP
    codes, `scales` a non-empty contiguous finite non-negative float32 tensor whose doubling must
    not overflow.  The returned bytes are Gaudi2 half-range codes in float8_e4m3fn storage.
    """
    if (not isinstance(weight, torch.Tensor) or weight.dtype != torch.float8_e4m3fn
            or not weight.is_contiguous() or not weight.numel() or weight.requires_grad):
        raise ValueError("expected a nonempty contiguous E4M3FN weight")
    if (not isinstance(scales, torch.Tensor) or scales.dtype != torch.float32
            or not scales.is_contiguous() or not scales.numel() or scales.requires_grad):
        raise ValueError("expected nonempty contiguous finite nonnegative FP32 scales")
    lib = _lib.load()
    dev = _device_for(weight, scales)
    on_host = weight.device.type == "cpu"
    with torch.cuda.device(dev):
        w = weight.to(dev, non_blocking=True)
        s = scales.to(dev, non_blocking=True)
        enc = torch.empty_like(w)
        adj = torch.empty_like(s)
        st = _status_buffer(dev)
        rc = lib.bfp8_reencode_half(w.data_ptr(), enc.data_ptr(), w.numel(), s.data_ptr(), adj.data_ptr(),
                                    s.numel(), st.data_ptr(), st.data_ptr() + 8, _stream_ptr())
        _lib.check(rc, "bfp8_reencode_half")
        rounded, status = _read_status(st)
    if status & _lib.STATUS_BAD_SCALE:
        raise ValueError("expected finite nonnegative FP32 scales whose doubling does not overflow FP32")
    if status & _lib.STATUS_NONFINITE_CODE:
        raise ValueError("nonfinite OCP E4M3FN checkpoint code")
    if on_host:
        enc, adj = enc.cpu(), adj.cpu()
    return enc, adj, rounded


def quantize_block128(w, native_half=False):
    """fp32 [R, C] -> (E4M3 codes [R, C] as float8_e4m3fn, fp32 scales [ceil(R/128), ceil(C/128)]).

    Per 128x128 tile: scale = max(amax, 1e-10) * fp32(1/448), code = RNE(clamp(w / scale, +-448)) -
    the rule of block_fp8_oracle.py:27-28 over a square tile.  With native_half the codes are
    additionally halved (RNE) and the scales doubled (:31-35) in the same pass, which is the
    format the Gaudi2-style GEMM consumes.
    """
    if not isinstance(w, torch.Tensor) or w.dtype != torch.float32 or w.ndim != 2 or not w.numel():
        raise ValueError("expected a nonempty 2-D FP32 tensor")
    if w.stride(1) != 1:
        raise ValueError("expected unit stride along the last dimension")
    lib = _lib.load()
    dev = _device_for(w)
    on_host = w.device.type == "cpu"
    with torch.cuda.device(dev):
        wd = w.to(dev, non_blocking=True)
        r, c = wd.shape
        codes = torch.empty((r, c), dtype=torch.uint8, device=dev)
        scales = torch.empty(((r + BLOCK - 1) // BLOCK, (c + BLOCK - 1) // BLOCK), dtype=torch.float32, device=dev)
        rc = lib.bfp8_quant_block128_f32(wd.data_ptr(), r, c, wd.stride(0), codes.data_ptr(), c,
                                         scales.data_ptr(), int(bool(native_half)), _stream_ptr())
        _lib.check(rc, "bfp8_quant_block128_f32")
    codes = codes.view(torch.float8_e4m3fn)
    if on_host:
        codes, scales = codes.cpu(), scales.cpu()
    return codes, scales


def quantize_act_1x128(x, native_half=False, check_finite=False):
    """bf16 [M, K] -> (E4M3 codes [M, K], fp32 scales [M, ceil(K/128)]).

    block_fp8_oracle.py:25-28 (and :31-34 with native_half).  The scales come back as an [M, G]
    view of group-major storage ([G, M] contiguous), the layout the GEMM epilogue reads.
    With check_finite an inf/NaN activation raises ValueError (block_fp8_oracle.py:22-24); the
    check costs one device synchronisation.
    """
    if not isinstance(x, torch.Tensor) or x.dtype != torch.bfloat16 or x.ndim != 2 or not x.numel():
        raise ValueError("expected a nonempty 2-D BF16 tensor")
    if x.stride(1) != 1:
        raise ValueError("expected unit stride along the last dimension")
    lib = _lib.load()
    dev = _device_for(x)
    on_host = x.device.type == "cpu"
    with torch.cuda.device(dev):
        xd = x.to(dev, non_blocking=True)
        m, k = xd.shape
        g = (k + BLOCK - 1) // BLOCK
        codes = torch.empty((m, k), dtype=torch.uint8, device=dev)
        scales_gm = torch.empty((g, m), dtype=torch.float32, device=dev)
        st = _status_buffer(dev) if check_finite else None
        rc = lib.bfp8_quant_act_1x128_bf16(xd.data_ptr(), m, k, xd.stride(0), codes.data_ptr(), k,
                                           scales_gm.data_ptr(), 1, m, int(bool(native_half)),
                                           st.data_ptr() + 8 if check_finite else None, _stream_ptr())
        _lib.check(rc, "bfp8_quant_act_1x128_bf16")
        if check_finite and _read_status(st)[1] & _lib.STATUS_NONFINITE_INPUT:
            raise ValueError("finite original inputs required")
    codes = codes.view(torch.float8_e4m3fn)
    scales = scales_gm.t()
    if on_host:
        codes, scales = codes.cpu(), scales.cpu()
    return codes, scales



def silu_quantize_act_1x128(gate_up, native_half=False):
    """bf16 [M, 2 * I] (gate columns, then up columns) -> (E4M3 codes [M, I], fp32 scales [M, ceil(I/128)]).

    gk_silu_and_mul_bf16_v1 (csrc/tpc/generic_dense/silu_and_mul_bf16.c:16) and the 1x128 quantizer of
    block_fp8_oracle.py:25-28 in one kernel: the same codes and scales as
    quantize_act_1x128(silu_and_mul(gate_up)), without writing and re-reading the [M, I] product.
    """
    if (not isinstance(gate_up, torch.Tensor) or gate_up.dtype != torch.bfloat16 or gate_up.ndim != 2
            or gate_up.shape[1] % 2 or not gate_up.numel() or gate_up.stride(1) != 1 or gate_up.device.type != "cuda"):
        raise ValueError("expected a nonempty bf16 [M, 2 * I] CUDA tensor with unit column stride")
    lib = _lib.load()
    dev = gate_up.device
    m, inter = gate_up.shape[0], gate_up.shape[1] // 2
    g = (inter + BLOCK - 1) // BLOCK
    with torch.cuda.device(dev):
        codes = torch.empty((m, inter), dtype=torch.uint8, device=dev)
        scales_gm = torch.empty((g, m), dtype=torch.float32, device=dev)
        rc = lib.bfp8_silu_quant_act_1x128_bf16(gate_up.data_ptr(), m, inter, gate_up.stride(0), codes.data_ptr(), inter,
                                                scales_gm.data_ptr(), 1, m, int(bool(native_half)), None, _stream_ptr())
        _lib.check(rc, "bfp8_silu_quant_act_1x128_bf16")
    return codes.view(torch.float8_e4m3fn), scales_gm.t()

def quantize_act_token(x, native_half=True, check_finite=False):
    """bf16 [M, K] -> (E4M3 codes [M, K], fp32 scales [M]): one scale per row.

    The per-token quantizer of the reference's per-token / per-channel FP8 variant
    (csrc/tpc/block_fp8_framework/activation_token.c:4-26): scale = amax / 448 over the whole row (1 for an
    all-zero row), code = RNE(x / scale); with native_half (that kernel's only mode) the codes are halved and
    the stored scale doubled.
    """
    if not isinstance(x, torch.Tensor) or x.dtype != torch.bfloat16 or x.ndim != 2 or not x.numel():
        raise ValueError("expected a nonempty 2-D BF16 tensor")
    if x.stride(1) != 1:
        raise ValueError("expected unit stride along the last dimension")
    lib = _lib.load()
    dev = _device_for(x)
    on_host = x.device.type == "cpu"
    with torch.cuda.device(dev):
        xd = x.to(dev, non_blocking=True)
        m, k = xd.shape
        codes = torch.empty((m, k), dtype=torch.uint8, device=dev)
        scales = torch.empty((m,), dtype=torch.float32, device=dev)
        st = _status_buffer(dev) if check_finite else None
        rc = lib.bfp8_quant_act_token_bf16(xd.data_ptr(), m, k, xd.stride(0), codes.data_ptr(), k, scales.data_ptr(),
                                           int(bool(native_half)), st.data_ptr() + 8 if check_finite else None,
                                           _stream_ptr())
        _lib.check(rc, "bfp8_quant_act_token_bf16")
        if check_finite and _read_status(st)[1] & _lib.STATUS_NONFINITE_INPUT:
            raise ValueError("finite original inputs required")
    codes = codes.view(torch.float8_e4m3fn)
    if on_host:
        codes, scales = codes.cpu(), scales.cpu()
    return codes, scales


def decode_e4m3(codes, scales, out_dtype=torch.float32):
    """value(code) * 128x128 block scale -> fp32 or bf16 [R, C].

    value() is the E4M3 decode of the reference's tests/test_fp8_codec.py:8-12 (identical for OCP
    codes and for Gaudi2 half-range codes up to magnitude 0x77).
    """
    if (not isinstance(codes, torch.Tensor) or codes.dtype not in (torch.float8_e4m3fn, torch.uint8)
            or codes.ndim != 2 or not codes.numel() or not codes.is_contiguous()):
        raise ValueError("expected a nonempty contiguous 2-D E4M3 code tensor")
    r, c = codes.shape
    if (not isinstance(scales, torch.Tensor) or scales.dtype != torch.float32 or not scales.is_contiguous()
            or tuple(scales.shape) != ((r + BLOCK - 1) // BLOCK, (c + BLOCK - 1) // BLOCK)):
        raise ValueError("block128 scale grid mismatch")
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("out_dtype must be float32 or bfloat16")
    lib = _lib.load()
    dev = _device_for(codes, scales)
    on_host = codes.device.type == "cpu"
    with torch.cuda.device(dev):
        cd = codes.to(dev, non_blocking=True)
        sd = scales.to(dev, non_blocking=True)
        out = torch.empty((r, c), dtype=out_dtype, device=dev)
        rc = lib.bfp8_decode_block128(cd.data_ptr(), r, c, c, sd.data_ptr(), out.data_ptr(),
                                      _lib.OUT_BF16 if out_dtype == torch.bfloat16 else _lib.OUT_F32, c,
                                      _stream_ptr())
        _lib.check(rc, "bfp8_decode_block128")
    return out.cpu() if on_host else out
