"""Load-time pipeline: stream a block-FP8 checkpoint from host memory onto the GPU in the kernel's format.

The reference's loader calls `reencode_e4m3fn_half` tensor by tensor on the CPU
(python/gaudi_kernels/fp8_codec.py:14-53, "layout packing is a separate step", :19) and then repacks
each weight K-block-major for the Gaudi2 MME (`[G, N, 128]`, tests/fp8_hybrid_tpcsim_test.cpp:223).
On B200 the tcgen05 kernels read the checkpoint's own row-major `[N, K]` layout - one 128-code K block of a
row is one 128-byte shared-memory row - so the only format work left is the half-range re-encode (and,
for a fused gate/up weight, the 64-row interleave of the SwiGLU kernel).  What is worth pipelining is the
host-to-device copy: `stream_checkpoint` stages tensor t + 1 into pinned memory and copies it over PCIe on
a side stream while tensor t is re-encoded, and reads all status words once at the end.

Every check of `reencode_e4m3fn_half` still applies (0x7f / 0xff codes, scales that are negative or
non-finite, and - where the scales are doubled, native_half=True - scales that overflow when doubled);
a violation raises ValueError naming the tensor.  With native_half=False the codes are kept as they are and
a read-only kernel (bfp8_validate_e4m3) makes the checks.
"""

import torch

from . import _lib
from .fp8_codec import BLOCK, _stream_ptr


class _Staging:
    """Two pinned host buffers and two device buffers used alternately.

    A host buffer is rewritten only after the copy out of it has finished; a device buffer only after the
    re-encode that read it has finished (the copy stream waits for that event, the host does not).
    """

    def __init__(self, nbytes, device):
        self.device = device
        self.host = [torch.empty(nbytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.dev = [None, None]
        self.copied = [None, None]         # event on the copy stream: the host buffer may be rewritten
        self.consumed = [None, None]       # event on the main stream: the device buffer may be rewritten
        self.turn = 0

    def take(self, host_bytes, dev_bytes, copy_stream):
        i = self.turn
        self.turn ^= 1
        if self.copied[i] is not None:
            self.copied[i].synchronize()
        if self.host[i].numel() < host_bytes:
            self.host[i] = torch.empty(host_bytes, dtype=torch.uint8).pin_memory()
        if dev_bytes and (self.dev[i] is None or self.dev[i].numel() < dev_bytes):
            if self.consumed[i] is not None:
                self.consumed[i].synchronize()             # the old buffer goes back to the allocator
            with torch.cuda.stream(copy_stream):
                self.dev[i] = torch.empty(dev_bytes, dtype=torch.uint8, device=self.device)
            self.dev[i].record_stream(torch.cuda.current_stream())      # read by kernels on the caller's stream
        elif dev_bytes and self.consumed[i] is not None:
            copy_stream.wait_event(self.consumed[i])
        return i


def _round_up(x, a):
    return (x + a - 1) // a * a


def _check_entry(name, weight, scales):
    if (not isinstance(weight, torch.Tensor) or weight.dtype not in (torch.float8_e4m3fn, torch.uint8)
            or weight.ndim != 2 or not weight.is_contiguous() or not weight.numel() or weight.device.type != "cpu"):
        raise ValueError("%s: expected a nonempty contiguous 2-D E4M3FN host weight" % name)
    grid = ((weight.shape[0] + BLOCK - 1) // BLOCK, (weight.shape[1] + BLOCK - 1) // BLOCK)
    if (not isinstance(scales, torch.Tensor) or scales.dtype != torch.float32 or not scales.is_contiguous()
            or tuple(scales.shape) != grid or scales.device.type != "cpu"):
        raise ValueError("%s: original block128 scale grid mismatch" % name)


def stream_checkpoint(entries, device=None, native_half=True, swiglu=(), staging_bytes=64 << 20):
    """Copy and re-encode weights; returns {name: (codes float8_e4m3fn [N, K'], scales fp32, rounded count)}.

    entries        iterable of (name, weight, scales): host tensors, weight float8_e4m3fn / uint8 [N, K] of OCP
                   codes, scales fp32 [ceil(N/128), ceil(K/128)] - consumed lazily, so a generator that reads one
                   tensor at a time from disk keeps host memory at one tensor
    native_half    re-encode to the half range and double the scales (fp8_codec.py:30-40); False keeps OCP codes
    swiglu         names of fused gate/up weights [2 I, K] to interleave for gemm_block_fp8_swiglu
                   (K' is K rounded up to 16 for those, K otherwise)
    staging_bytes  initial size of each of the two pinned staging buffers (they grow to the largest tensor)
    """
    if device is None:
        if not torch.cuda.is_available():
            raise _lib.Bfp8Error("a CUDA device is required; this package has no CPU path")
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    lib = _lib.load()
    swiglu = set(swiglu)
    out, order = {}, []
    with torch.cuda.device(device):
        main = torch.cuda.current_stream()
        copy = torch.cuda.Stream(device=device)
        staging = _Staging(staging_bytes, device)
        status_rows = []
        for name, weight, scales in entries:
            _check_entry(name, weight, scales)
            if name in out:
                raise ValueError("%s: duplicate tensor name" % name)
            n, k = weight.shape
            raw = weight.view(torch.uint8).view(-1)
            w_bytes, s_bytes = raw.numel(), scales.numel() * 4
            # pinned staging slot: [weight bytes unless the source is pinned already | scales]; the scales always
            # go through it, because a copy from pageable memory would make the host wait for the copy stream
            w_stage = 0 if raw.is_pinned() else _round_up(w_bytes, 256)
            # device staging slot (only when the bytes are transformed on the way): [weight | scales]
            d_scales_at = _round_up(w_bytes, 256)
            slot = staging.take(w_stage + s_bytes, d_scales_at + s_bytes if native_half else 0, copy)
            hbuf = staging.host[slot]
            if w_stage:
                hbuf[:w_bytes].copy_(raw)                          # pageable -> pinned on the host
            hbuf[w_stage:w_stage + s_bytes].view(torch.float32).copy_(scales.view(-1))
            host_w = hbuf[:w_bytes] if w_stage else raw
            host_s = hbuf[w_stage:w_stage + s_bytes].view(torch.float32)
            dev_w = torch.empty((n, k), dtype=torch.uint8, device=device)
            dev_s = torch.empty(scales.shape, dtype=torch.float32, device=device)
            st = torch.zeros(4, dtype=torch.int32, device=device)
            if native_half:
                dbuf = staging.dev[slot]
                raw_w = dbuf[:w_bytes]
                raw_s = dbuf[d_scales_at:d_scales_at + s_bytes].view(torch.float32)
                with torch.cuda.stream(copy):
                    raw_w.copy_(host_w, non_blocking=True)
                    raw_s.copy_(host_s, non_blocking=True)
                    landed = torch.cuda.Event()
                    landed.record(copy)
                staging.copied[slot] = landed
                main.wait_event(landed)
                rc = lib.bfp8_reencode_half(raw_w.data_ptr(), dev_w.data_ptr(), w_bytes, raw_s.data_ptr(),
                                            dev_s.data_ptr(), scales.numel(), st.data_ptr(), st.data_ptr() + 8,
                                            _stream_ptr())
                _lib.check(rc, "bfp8_reencode_half")
                consumed = torch.cuda.Event()
                consumed.record(main)
                staging.consumed[slot] = consumed
            else:
                # straight into the resident tensors; the copy stream first waits for whatever `main` last did
                # with the memory the allocator just handed out
                ready = torch.cuda.Event()
                ready.record(main)
                copy.wait_event(ready)
                with torch.cuda.stream(copy):
                    dev_w.view(-1).copy_(host_w, non_blocking=True)
                    dev_s.view(-1).copy_(host_s, non_blocking=True)
                    landed = torch.cuda.Event()
                    landed.record(copy)
                staging.copied[slot] = landed
                main.wait_event(landed)
                dev_w.record_stream(copy)
                dev_s.record_stream(copy)
                # the codes stay as they are, the checks of fp8_codec.py:25-29,48-49 still apply
                rc = lib.bfp8_validate_e4m3(dev_w.data_ptr(), w_bytes, dev_s.data_ptr(), scales.numel(),
                                            st.data_ptr() + 8, _stream_ptr())
                _lib.check(rc, "bfp8_validate_e4m3")
            if name in swiglu:
                if n % (2 * BLOCK) != 0:
                    raise ValueError("%s: fused gate/up weight must be [2 * I, K] with I a multiple of 128" % name)
                src = dev_w if k % 16 == 0 else torch.nn.functional.pad(dev_w, (0, (k + 15) // 16 * 16 - k))
                dst = torch.empty_like(src)
                rc = lib.bfp8_swiglu_interleave_weight(src.data_ptr(), src.stride(0), dst.data_ptr(), dst.stride(0),
                                                       n // 2, src.shape[1], _stream_ptr())
                _lib.check(rc, "bfp8_swiglu_interleave_weight")
                dev_w = dst
            out[name] = (dev_w.view(torch.float8_e4m3fn), dev_s)
            order.append(name)
            status_rows.append(st)
        if not order:
            return {}
        host_status = torch.stack(status_rows).cpu()               # one synchronisation for the whole checkpoint
    result = {}
    for name, row in zip(order, host_status):
        lo, hi, status = int(row[0]) & 0xFFFFFFFF, int(row[1]) & 0xFFFFFFFF, int(row[2]) & 0xFFFFFFFF
        if status & _lib.STATUS_BAD_SCALE:
            raise ValueError("%s: expected finite nonnegative FP32 scales whose doubling does not overflow FP32" % name)
        if status & _lib.STATUS_NONFINITE_CODE:
            raise ValueError("%s: nonfinite OCP E4M3FN checkpoint code" % name)
        codes, scales = out[name]
        result[name] = (codes, scales, (hi << 32) | lo)
    return result
