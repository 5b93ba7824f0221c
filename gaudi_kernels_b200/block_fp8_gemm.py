"""Block-scaled E4M3 GEMM on B200 behind the reference oracle's signature.

`reference(x, weight, scales, *, native_half=False, bias=None)` takes the arguments of
python/gaudi_kernels/block_fp8_oracle.py:11 of tracycam/gaudi-kernels - bf16 activations, the
original OCP float8_e4m3fn weight [N, K] and its fp32 128x128 scale grid - and returns the bf16
product, computed by libbfp8.so's kernels: 1x128 activation quantization (:25-28), optional
half-range adaptation of both operands (:31-35), the per-K-block contraction on the tensor cores
and the fp32 scale promotion (:38-41), bias (:42-45), bf16 rounding (:46).  Differences from the
reference, all relaxations: any number of activation rows (the reference insists on one, :16-17),
and tensors may live on a CUDA device.  Contract breaches raise ValueError as there.

`gemm_block_fp8` is the hot path for operands that are already quantized (weights are prepared
once at load time; the reference's loader does that with fp8_codec.reencode_e4m3fn_half).
There is no CPU implementation in this package.
"""

import torch

from . import _lib
from .fp8_codec import BLOCK, _device_for, _read_status, _status_buffer, _stream_ptr, quantize_act_1x128

# Zero-initialised scratch per (device, stream).  The small-M schedule keeps per-tile arrival counters
# there and returns them to zero, so one buffer serves every call issued on that stream.
_workspaces = {}


def _workspace(dev, nbytes):
    key = (dev.index, _stream_ptr())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1), dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


_HOST_ROW_BLOCK = 1024          # reference() on host tensors pipelines blocks of at least this many rows
_HOST_MAX_BLOCKS = 8            # finer blocks change nothing: the copy back to the host is the bound
_copy_streams = {}


def _copy_stream(dev):
    """A second stream per device for copying results back while the next block is computed."""
    st = _copy_streams.get(dev.index)
    if st is None:
        st = torch.cuda.Stream(device=dev)
        _copy_streams[dev.index] = st
    return st


_WAIT_TIMEOUT_MSG = "a bounded wait inside the GEMM kernel expired (BFP8_STATUS_WAIT_TIMEOUT); output is invalid"


def _group_major(a_scales, m, g):
    """Return (tensor, ldsa) with element (row i, group g) at data[g * ldsa + i]."""
    if tuple(a_scales.shape) != (m, g) or a_scales.dtype != torch.float32:
        raise ValueError("activation scales must be FP32 [M, ceil(K/128)]")
    if m == 1 or g == 1:
        a_scales = a_scales.contiguous() if not a_scales.is_contiguous() else a_scales
        return a_scales, m
    if a_scales.stride(0) == 1 and a_scales.stride(1) >= m:
        return a_scales, a_scales.stride(1)
    t = a_scales.t().contiguous()          # [G, M]
    return t, m


def wait_timed_out(status):
    """True if a kernel given `status` (a tensor from new_status()) reported an expired bounded wait.

    Reads the word back (one synchronisation with the launching stream).  After a time-out the small-M schedule's
    arrival counters may be non-zero, so the cached workspaces are dropped; the outputs of the calls that shared
    the status word are invalid.
    """
    timed_out = bool(_read_status(status)[1] & _lib.STATUS_WAIT_TIMEOUT)
    if timed_out:
        _workspaces.clear()
    return timed_out


def new_status(device):
    """A zeroed device status buffer for gemm_block_fp8(..., check=False, status=...); poll it with wait_timed_out."""
    return _status_buffer(device)


def set_weights_at_rest(on):
    """Tell the library whether the weight codes given to the decode-bucket GEMMs (M <= 128) are at rest, i.e. written
    by nothing that is still in flight when a GEMM is enqueued (bfp8_set_weights_at_rest).  When they are, each GEMM
    starts streaming its weight before the previous kernel of the stream has finished; results are unchanged.
    Process-wide; returns the previous setting.  A serving process turns it on once its checkpoint is loaded and
    the device synchronised, and off again around any in-place rewrite of a weight."""
    return bool(_lib.load().bfp8_set_weights_at_rest(1 if on else 0))


def gemm_block_fp8(a_codes, a_scales, w_codes, w_scales, bias=None, out=None, out_dtype=torch.bfloat16,
                   check=True, schedule=0, max_ctas=0, wait_limit_cycles=0, status=None):
    """out[i, j] = sum_g a_scales[i, g] * w_scales[j // 128, g] * <a_codes[i, g-block], w_codes[j, g-block]> (+ bias[j]).

    a_codes  E4M3 [M, K] (float8_e4m3fn or uint8), contiguous, on a CUDA device
    a_scales fp32 [M, G]; group-major storage (as returned by quantize_act_1x128) avoids a copy
    w_codes  E4M3 [N, K], contiguous;  w_scales fp32 [ceil(N/128), G] contiguous
    bias     fp32 [N] or None;  out_dtype torch.bfloat16 (default) or torch.float32
    check    read the device status word after the launch (one synchronisation) and raise if a
             bounded wait expired; pass False on a latency-critical path together with `status`
    status   a buffer from new_status() that receives the kernel's status bits; several calls may share one.
             With check=False the caller reads it later through wait_timed_out(status).  Without a status
             buffer an unchecked call cannot report an expired wait.
    """
    for name, t in (("a_codes", a_codes), ("w_codes", w_codes)):
        if (not isinstance(t, torch.Tensor) or t.dtype not in (torch.float8_e4m3fn, torch.uint8) or t.ndim != 2
                or not t.is_contiguous() or t.device.type != "cuda"):
            raise ValueError("%s must be a contiguous 2-D E4M3 tensor on a CUDA device" % name)
    m, k = a_codes.shape
    n = w_codes.shape[0]
    if w_codes.shape[1] != k or m < 1 or n < 1 or k < 1:
        raise ValueError("a_codes [M, K] and w_codes [N, K] must share K")
    g = (k + BLOCK - 1) // BLOCK
    if (not isinstance(w_scales, torch.Tensor) or w_scales.dtype != torch.float32 or not w_scales.is_contiguous()
            or tuple(w_scales.shape) != ((n + BLOCK - 1) // BLOCK, g)):
        raise ValueError("original block128 scale grid mismatch")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("out_dtype must be bfloat16 or float32")
    dev = a_codes.device
    if bias is not None:
        if bias.numel() != n:
            raise ValueError("bias with N elements required")
        bias = bias.to(device=dev, dtype=torch.float32).contiguous().view(-1)
    lib = _lib.load()
    with torch.cuda.device(dev):
        if k % 16 != 0:
            # TMA needs 16-byte row pitches: pad K with zero codes (zero contributes nothing).
            kp = (k + 15) // 16 * 16
            a_codes = torch.nn.functional.pad(a_codes.view(torch.uint8), (0, kp - k))
            w_codes = torch.nn.functional.pad(w_codes.view(torch.uint8), (0, kp - k))
        lda, ldw = a_codes.stride(0), w_codes.stride(0)
        sa, ldsa = _group_major(a_scales.to(dev), m, g)
        w_scales = w_scales.to(dev)
        if out is None:
            ldo = n if out_dtype == torch.float32 else (n + 7) // 8 * 8
            storage = torch.empty((m, ldo), dtype=out_dtype, device=dev)
            out = storage[:, :n]
        else:
            if (out.dtype != out_dtype or tuple(out.shape) != (m, n) or out.stride(1) != 1
                    or out.device != dev):
                raise ValueError("out must be [M, N] of out_dtype with unit column stride on the operand device")
            ldo = out.stride(0)
        ws_bytes = lib.bfp8_gemm_block128_workspace_bytes(m, n, k)
        ws = _workspace(dev, ws_bytes) if ws_bytes else None
        st = status if status is not None else _status_buffer(dev)
        rc = lib.bfp8_gemm_block128_ex(
            a_codes.data_ptr(), lda, sa.data_ptr(), ldsa, w_codes.data_ptr(), ldw, w_scales.data_ptr(),
            bias.data_ptr() if bias is not None else None, out.data_ptr(),
            _lib.OUT_BF16 if out_dtype == torch.bfloat16 else _lib.OUT_F32, ldo, m, n, k,
            ws.data_ptr() if ws is not None else None, ws_bytes, st.data_ptr() + 8, _stream_ptr(),
            schedule, max_ctas, wait_limit_cycles)
        _lib.check(rc, "bfp8_gemm_block128")
        if check and _read_status(st)[1] & _lib.STATUS_WAIT_TIMEOUT:
            _workspaces.clear()            # counters may have been left non-zero
            raise _lib.Bfp8Error(_WAIT_TIMEOUT_MSG)
    return out


def gemm_token_channel_fp8(a_codes, a_scales, w_codes, w_scales, bias=None, out=None, out_dtype=torch.bfloat16,
                           check=True):
    """out[i, j] = <a_codes[i], w_codes[j]> * a_scales[i] * w_scales[j] (+ bias[j]): per-token / per-channel scales.

    The reference's per-token / per-channel FP8 variant (gk_fp8_token_quant_bf16_v1 -> MME GEMM ->
    gk_fp8_channel_finish_bf16_v1, csrc/tpc/block_fp8_framework/channel_finish.c:2-18) as one kernel.
    a_codes E4M3 [M, K], a_scales fp32 [M], w_codes E4M3 [N, K], w_scales fp32 [N], all on one CUDA device.
    """
    for name, t in (("a_codes", a_codes), ("w_codes", w_codes)):
        if (not isinstance(t, torch.Tensor) or t.dtype not in (torch.float8_e4m3fn, torch.uint8) or t.ndim != 2
                or not t.is_contiguous() or t.device.type != "cuda"):
            raise ValueError("%s must be a contiguous 2-D E4M3 tensor on a CUDA device" % name)
    m, k = a_codes.shape
    n = w_codes.shape[0]
    if w_codes.shape[1] != k or m < 1 or n < 1 or k < 1:
        raise ValueError("a_codes [M, K] and w_codes [N, K] must share K")
    if a_scales.dtype != torch.float32 or a_scales.numel() != m or w_scales.dtype != torch.float32 or w_scales.numel() != n:
        raise ValueError("a_scales must be FP32 [M] and w_scales FP32 [N]")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("out_dtype must be bfloat16 or float32")
    dev = a_codes.device
    if bias is not None:
        if bias.numel() != n:
            raise ValueError("bias with N elements required")
        bias = bias.to(device=dev, dtype=torch.float32).contiguous().view(-1)
    lib = _lib.load()
    with torch.cuda.device(dev):
        if k % 16 != 0:
            kp = (k + 15) // 16 * 16
            a_codes = torch.nn.functional.pad(a_codes.view(torch.uint8), (0, kp - k))
            w_codes = torch.nn.functional.pad(w_codes.view(torch.uint8), (0, kp - k))
        a_scales = a_scales.to(dev).contiguous().view(-1)
        w_scales = w_scales.to(dev).contiguous().view(-1)
        if out is None:
            ldo = n if out_dtype == torch.float32 else (n + 7) // 8 * 8
            out = torch.empty((m, ldo), dtype=out_dtype, device=dev)[:, :n]
        else:
            if out.dtype != out_dtype or tuple(out.shape) != (m, n) or out.stride(1) != 1 or out.device != dev:
                raise ValueError("out must be [M, N] of out_dtype with unit column stride on the operand device")
            ldo = out.stride(0)
        st = _status_buffer(dev)
        rc = lib.bfp8_gemm_token_channel(
            a_codes.data_ptr(), a_codes.stride(0), a_scales.data_ptr(), w_codes.data_ptr(), w_codes.stride(0),
            w_scales.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(),
            _lib.OUT_BF16 if out_dtype == torch.bfloat16 else _lib.OUT_F32, ldo, m, n, k, st.data_ptr() + 8, _stream_ptr())
        _lib.check(rc, "bfp8_gemm_token_channel")
        if check and _read_status(st)[1] & _lib.STATUS_WAIT_TIMEOUT:
            raise _lib.Bfp8Error(_WAIT_TIMEOUT_MSG)
    return out


def prepare_weight(weight, scales, native_half=True):
    """Load-time weight preparation: OCP codes + scales -> what gemm_block_fp8 consumes.

    With native_half this is fp8_codec.reencode_e4m3fn_half (python/gaudi_kernels/fp8_codec.py:14-53)
    on the GPU; otherwise the OCP codes are used as they are.  Returns (codes, scales) on the device.
    """
    from .fp8_codec import reencode_e4m3fn_half
    dev = _device_for(weight, scales)
    weight, scales = weight.to(dev), scales.to(dev)
    if native_half:
        weight, scales, _ = reencode_e4m3fn_half(weight, scales)
    return weight, scales


def prepare_weight_swiglu(weight, scales, native_half=True):
    """Load-time preparation of a fused gate/up weight for gemm_block_fp8_swiglu.

    weight float8_e4m3fn / uint8 [2 * I, K] with the gate projection in rows [0, I) and the up projection in
    rows [I, 2 * I) (the order csrc/tpc/generic_dense/silu_and_mul_bf16.c:29 reads); scales fp32 [2 * I / 128, G].
    Re-encodes to the half range when asked (as prepare_weight), then interleaves the rows in chunks of 64
    so a GEMM tile holds both factors of its outputs.  The scale grid keeps its order.  I % 128 == 0.
    """
    codes, scales = prepare_weight(weight, scales, native_half)
    if codes.ndim != 2 or codes.shape[0] % (2 * BLOCK) != 0:
        raise ValueError("fused gate/up weight must be [2 * I, K] with I a multiple of 128")
    inter, k = codes.shape[0] // 2, codes.shape[1]
    dev = codes.device
    lib = _lib.load()
    with torch.cuda.device(dev):
        src = codes.contiguous().view(torch.uint8)
        if k % 16 != 0:
            src = torch.nn.functional.pad(src, (0, (k + 15) // 16 * 16 - k))
        dst = torch.empty_like(src)
        rc = lib.bfp8_swiglu_interleave_weight(src.data_ptr(), src.stride(0), dst.data_ptr(), dst.stride(0), inter,
                                               src.shape[1], _stream_ptr())
        _lib.check(rc, "bfp8_swiglu_interleave_weight")
    return dst.view(torch.float8_e4m3fn), scales


def gemm_block_fp8_swiglu(a_codes, a_scales, w_codes, w_scales, bias=None, out=None, check=True, small_m=True):
    """bf16 [M, I] = silu(gate) * up, with gate | up = the block-scaled GEMM of gemm_block_fp8 rounded to bf16.

    The gate/up GEMM and gk_silu_and_mul_bf16_v1 (csrc/tpc/generic_dense/silu_and_mul_bf16.c:16) as one
    kernel.  w_codes [2 * I, K'] and w_scales [2 * I / 128, G] come from prepare_weight_swiglu (K' is K
    rounded up to 16); bias fp32 [2 * I] in the fused weight's original order, or None.  With M <= 128 the
    weight-streaming (decode bucket) schedule runs on the same interleaved weight; small_m=False keeps the
    large-tile schedule for every M.
    """
    for name, t in (("a_codes", a_codes), ("w_codes", w_codes)):
        if (not isinstance(t, torch.Tensor) or t.dtype not in (torch.float8_e4m3fn, torch.uint8) or t.ndim != 2
                or not t.is_contiguous() or t.device.type != "cuda"):
            raise ValueError("%s must be a contiguous 2-D E4M3 tensor on a CUDA device" % name)
    m, k = a_codes.shape
    n2 = w_codes.shape[0]
    if n2 % (2 * BLOCK) != 0 or m < 1 or k < 1 or w_codes.shape[1] != (k + 15) // 16 * 16:
        raise ValueError("w_codes must be the [2 * I, K] output of prepare_weight_swiglu, I a multiple of 128")
    inter = n2 // 2
    g = (k + BLOCK - 1) // BLOCK
    if (not isinstance(w_scales, torch.Tensor) or w_scales.dtype != torch.float32 or not w_scales.is_contiguous()
            or tuple(w_scales.shape) != (n2 // BLOCK, g)):
        raise ValueError("original block128 scale grid mismatch")
    dev = a_codes.device
    if bias is not None:
        if bias.numel() != n2:
            raise ValueError("bias with 2 * I elements required")
        bias = bias.to(device=dev, dtype=torch.float32).contiguous().view(-1)
    lib = _lib.load()
    with torch.cuda.device(dev):
        if k % 16 != 0:
            a_codes = torch.nn.functional.pad(a_codes.view(torch.uint8), (0, w_codes.shape[1] - k))
        sa, ldsa = _group_major(a_scales.to(dev), m, g)
        w_scales = w_scales.to(dev)
        if out is None:
            out = torch.empty((m, inter), dtype=torch.bfloat16, device=dev)
        elif (out.dtype != torch.bfloat16 or tuple(out.shape) != (m, inter) or out.stride(1) != 1 or out.device != dev):
            raise ValueError("out must be bf16 [M, I] with unit column stride on the operand device")
        st = _status_buffer(dev)
        ws_bytes = lib.bfp8_gemm_block128_workspace_bytes(m, n2, w_codes.shape[1]) if (small_m and m <= 128) else 0
        ws = _workspace(dev, ws_bytes) if ws_bytes else None
        rc = lib.bfp8_gemm_block128_swiglu(
            a_codes.data_ptr(), a_codes.stride(0), sa.data_ptr(), ldsa, w_codes.data_ptr(), w_codes.stride(0),
            w_scales.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(), out.stride(0),
            m, inter, w_codes.shape[1], ws.data_ptr() if ws is not None else None, ws_bytes, st.data_ptr() + 8,
            _stream_ptr())
        _lib.check(rc, "bfp8_gemm_block128_swiglu")
        if check and _read_status(st)[1] & _lib.STATUS_WAIT_TIMEOUT:
            _workspaces.clear()
            raise _lib.Bfp8Error(_WAIT_TIMEOUT_MSG)
    return out


def silu_and_mul(gate_up, out=None):
    """bf16 [rows, 2 * I] (gate columns, then up columns) -> bf16 [rows, I] = silu(gate) * up.

    gk_silu_and_mul_bf16_v1 (csrc/tpc/generic_dense/silu_and_mul_bf16.c:16) as a stand-alone kernel, for GEMM
    results of the small-M schedule; gemm_block_fp8_swiglu fuses the same step for large M.
    """
    if (not isinstance(gate_up, torch.Tensor) or gate_up.dtype != torch.bfloat16 or gate_up.ndim != 2
            or gate_up.shape[1] % 2 or not gate_up.numel() or gate_up.stride(1) != 1 or gate_up.device.type != "cuda"):
        raise ValueError("expected a nonempty bf16 [rows, 2 * I] CUDA tensor with unit column stride")
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((rows, inter), dtype=torch.bfloat16, device=gate_up.device)
    elif (out.dtype != torch.bfloat16 or tuple(out.shape) != (rows, inter) or out.stride(1) != 1
          or out.device != gate_up.device):
        raise ValueError("out must be bf16 [rows, I] with unit column stride on the input's device")
    with torch.cuda.device(gate_up.device):
        rc = _lib.load().bfp8_silu_and_mul_bf16(gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(), out.stride(0),
                                                rows, inter, _stream_ptr())
    _lib.check(rc, "bfp8_silu_and_mul_bf16")
    return out


def reference(x, weight, scales, *, native_half=False, bias=None, out_dtype=torch.bfloat16, out=None):
    """Drop-in for gaudi_kernels.block_fp8_oracle.reference, computed on the GPU.

    x bf16 [M, K]; weight float8_e4m3fn [N, K] (original OCP codes); scales fp32 [ceil(N/128), ceil(K/128)].
    Host tensors are copied to the current CUDA device and the result is returned on the host
    (into `out` when given - a pinned [M, N] tensor makes that copy asynchronous up to the final wait).
    """
    if (not isinstance(x, torch.Tensor) or not isinstance(weight, torch.Tensor) or not isinstance(scales, torch.Tensor)
            or x.dtype != torch.bfloat16 or weight.dtype != torch.float8_e4m3fn
            or scales.dtype != torch.float32 or x.ndim != 2 or weight.ndim != 2
            or x.shape[0] < 1 or x.shape[1] != weight.shape[1]):
        raise ValueError("BF16 activation rows, original OCP FP8 weight and FP32 scales required")
    n, k = weight.shape
    groups = (k + BLOCK - 1) // BLOCK
    if tuple(scales.shape) != ((n + BLOCK - 1) // BLOCK, groups):
        raise ValueError("original block128 scale grid mismatch")
    if bias is not None and bias.numel() != n:
        raise ValueError("bias with N elements required")
    lib = _lib.load()
    dev = _device_for(x, weight, scales)
    on_host = x.device.type == "cpu"
    with torch.cuda.device(dev):
        wd = weight.to(dev, non_blocking=True).contiguous()
        sd = scales.to(dev, non_blocking=True).contiguous()
        st = _status_buffer(dev)
        if native_half:
            # weight side of block_fp8_oracle.py:31-35; also validates codes and scales
            enc = torch.empty_like(wd)
            sw = torch.empty_like(sd)
            rc = lib.bfp8_reencode_half(wd.data_ptr(), enc.data_ptr(), wd.numel(), sd.data_ptr(), sw.data_ptr(),
                                        sd.numel(), st.data_ptr(), st.data_ptr() + 8, _stream_ptr())
            _lib.check(rc, "bfp8_reencode_half")
        else:
            # block_fp8_oracle.py:22-24: the same rejections, without changing the codes
            enc, sw = wd, sd
            rc = lib.bfp8_validate_e4m3(wd.data_ptr(), wd.numel(), sd.data_ptr(), sd.numel(), st.data_ptr() + 8,
                                        _stream_ptr())
            _lib.check(rc, "bfp8_validate_e4m3")
        m = x.shape[0]

        def run_rows(x_rows, dev_out):
            """Quantize and multiply one block of activation rows (already on the device)."""
            mr = x_rows.shape[0]
            a_codes = torch.empty((mr, k), dtype=torch.uint8, device=dev)
            a_scales = torch.empty((groups, mr), dtype=torch.float32, device=dev)
            rc = lib.bfp8_quant_act_1x128_bf16(x_rows.data_ptr(), mr, k, x_rows.stride(0), a_codes.data_ptr(), k,
                                               a_scales.data_ptr(), 1, mr, int(bool(native_half)),
                                               st.data_ptr() + 8, _stream_ptr())
            _lib.check(rc, "bfp8_quant_act_1x128_bf16")
            return gemm_block_fp8(a_codes, a_scales.t(), enc, sw, bias=bias, out=dev_out, out_dtype=out_dtype,
                                  check=False, status=st)

        if not on_host:
            dev_out = out if (out is not None and out.device.type == "cuda") else None
            y = run_rows(x.to(dev).contiguous(), dev_out)
        else:
            if out is None:
                out = torch.empty((m, n), dtype=out_dtype)
            elif tuple(out.shape) != (m, n) or out.dtype != out_dtype:
                raise ValueError("out must be [M, N] of the output dtype")
            # Host tensors: the result (2 bytes per output) is larger than the inputs, so its copy back to the
            # host dominates.  Rows are processed in blocks and each block's result is copied on a second
            # stream while the next block is uploaded and multiplied (the two copy directions overlap).
            blocks = 1 if m < 2 * _HOST_ROW_BLOCK else min(_HOST_MAX_BLOCKS, m // _HOST_ROW_BLOCK)
            rows_per = ((m + blocks - 1) // blocks + BLOCK - 1) // BLOCK * BLOCK
            main = torch.cuda.current_stream()
            side = _copy_stream(dev)
            keep = []
            for r0 in range(0, m, rows_per):
                r1 = min(m, r0 + rows_per)
                xr = x[r0:r1].to(dev, non_blocking=True).contiguous()
                yr = run_rows(xr, None)
                done = torch.cuda.Event()
                done.record(main)
                side.wait_event(done)
                with torch.cuda.stream(side):
                    out[r0:r1].copy_(yr, non_blocking=True)
                keep.append((xr, yr))               # alive until the side stream has finished with them
            main.wait_stream(side)
            y = out
        status = _read_status(st)[1]               # synchronises: also completes the copy above
        if status & (_lib.STATUS_NONFINITE_CODE | _lib.STATUS_BAD_SCALE | _lib.STATUS_NONFINITE_INPUT):
            raise ValueError("finite original inputs required")
        if status & _lib.STATUS_WAIT_TIMEOUT:
            _workspaces.clear()            # arrival counters may have been left non-zero
            raise _lib.Bfp8Error(_WAIT_TIMEOUT_MSG)
    return y
