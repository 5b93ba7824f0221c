"""CPU restatement of the block-FP8 GEMM oracle, batched over rows. TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA GEMM: only the test-suite, the smoke
check and the CPU-baseline / reference legs of the benchmark may import it.  The
shipped package never does.

Follows python/gaudi_kernels/block_fp8_oracle.py:11-46 of tracycam/gaudi-kernels
step by step (validation :13-24, 1x128 activation quantization :25-28, zero-padded
weight :29-30, half-range adaptation :31-35, exact FP64 per-block dot :38-39,
scale promotion and FP64 sum over K blocks :40-41, bias :42-45, bf16 rounding :46).
The reference accepts one activation row per call (:16-17); this restatement takes
M rows and evaluates each row with the same operations in the same order, so a row
of its output equals the reference called on that row alone.  Parity is pinned by
fixtures generated from the reference itself (tests/golden/make_golden.py); the
reference ships no test of reference() of its own.

Third-party arithmetic: the RNE float8 cast and the FP64 matrix product are
torch's CPU operators (the reference pins no torch version; fixtures were made
with torch 2.11.0).
"""

import torch

BLOCK = 128


def _validate(x, weight, scales, bias):
    if (x.device.type != "cpu" or weight.device.type != "cpu" or scales.device.type != "cpu"
            or x.dtype != torch.bfloat16 or weight.dtype != torch.float8_e4m3fn
            or scales.dtype != torch.float32 or x.ndim != 2 or weight.ndim != 2
            or x.shape[0] < 1 or x.shape[1] != weight.shape[1]):
        raise ValueError("CPU BF16 activation rows, original OCP FP8 weight and FP32 scales required")
    n, k = weight.shape
    groups = (k + BLOCK - 1) // BLOCK
    if tuple(scales.shape) != ((n + BLOCK - 1) // BLOCK, groups):
        raise ValueError("original block128 scale grid mismatch")
    if not bool(torch.isfinite(x.float()).all() and torch.isfinite(weight.float()).all()
                and torch.isfinite(scales).all() and (scales >= 0).all()):
        raise ValueError("finite original inputs required")
    if bias is not None and (bias.device.type != "cpu" or bias.numel() != n):
        raise ValueError("CPU bias with N elements required")


class PreparedWeight:
    """Weight-side terms of block_fp8_oracle.py:29-35,38,40, computed once for many rows."""

    def __init__(self, weight, scales, native_half):
        n, k = weight.shape
        groups = (k + BLOCK - 1) // BLOCK
        w = torch.zeros((n, groups * BLOCK), dtype=torch.float32)
        w[:, :k] = weight.float()
        if native_half:
            w = (w * .5).to(torch.float8_e4m3fn).float()
            scales = scales * 2
        self.n, self.k, self.groups = n, k, groups
        self.native_half = native_half
        self.wg = w.reshape(n, groups, BLOCK).permute(1, 2, 0).double().contiguous()   # [G,128,N]
        self.sw = scales.repeat_interleave(BLOCK, dim=0)[:n].T.double().contiguous()    # [G,N]


def quantize_rows(x, groups, native_half):
    """block_fp8_oracle.py:25-28 (+ :31-34) for M rows: returns qa [M,G,128] f32, sa [M,G,1] f32."""
    m, k = x.shape
    a = torch.zeros((m, groups * BLOCK), dtype=torch.float32)
    a[:, :k] = x.float()
    a = a.view(m, groups, BLOCK)
    sa = a.abs().amax(-1, keepdim=True).clamp_min(1e-10) * (1.0 / 448.0)
    qa = (a / sa).clamp(-448, 448).to(torch.float8_e4m3fn).float()
    if native_half:
        qa = (qa * .5).to(torch.float8_e4m3fn).float()
        sa = sa * 2
    return qa, sa


def reference_rows(x, weight, scales, *, native_half=False, bias=None, chunk_rows=None,
                   prepared=None):
    """Returns (y_fp64 [M,N] before rounding, y_bf16 [M,N]).

    Rows are processed in chunks to bound the [G, rows, N] FP64 temporary.
    """
    _validate(x, weight, scales, bias)
    pw = prepared if prepared is not None else PreparedWeight(weight, scales, native_half)
    m = x.shape[0]
    if chunk_rows is None:
        chunk_rows = max(1, min(m, (256 << 20) // max(1, pw.groups * pw.n * 8)))
    y = torch.empty((m, pw.n), dtype=torch.float64)
    for r0 in range(0, m, chunk_rows):
        xr = x[r0:r0 + chunk_rows]
        qa, sa = quantize_rows(xr, pw.groups, native_half)
        # [G, rows, 128] x [G, 128, N]: every product and every 128-term sum is exact in FP64.
        partial = torch.bmm(qa.double().permute(1, 0, 2).contiguous(), pw.wg)          # [G,rows,N]
        sa_g = sa.double().permute(1, 0, 2)                                             # [G,rows,1]
        t = partial * sa_g * pw.sw.unsqueeze(1)
        y[r0:r0 + chunk_rows] = t.sum(0)
    if bias is not None:
        y = y + bias.double().view(1, -1)
    return y, y.to(torch.bfloat16)


def reference(x, weight, scales, *, native_half=False, bias=None):
    """Same signature and result as block_fp8_oracle.reference, for any number of rows."""
    return reference_rows(x, weight, scales, native_half=native_half, bias=bias)[1]


def w8a8_fp64_reference(x, weight, scales, bias=None):
    """The FP64 OCP W8A8 check of tests/fp8_hybrid_tpcsim_test.cpp:326-367, restated.

    Differs from reference() only in the activation scale: a true fp32 division
    amax/448 (:335) and 1.0 substituted for an all-zero group (:334).  Used for the
    reference's device gate (per-row relative L2 of bf16 outputs <= 0.01, :353-379).
    Returns bf16 [M,N].
    """
    m, k = x.shape
    n = weight.shape[0]
    groups = (k + BLOCK - 1) // BLOCK
    a = torch.zeros((m, groups * BLOCK), dtype=torch.float32)
    a[:, :k] = x.float()
    a = a.view(m, groups, BLOCK)
    amax = a.abs().amax(-1, keepdim=True)
    amax = torch.where(amax == 0, torch.ones_like(amax), amax)
    sa = amax / 448.0
    q = (a.abs() / sa).clamp(max=448.0).to(torch.float8_e4m3fn).double() * torch.sign(a).double()
    qx = (q * sa.double()).view(m, groups * BLOCK)[:, :k]
    sw = scales.repeat_interleave(BLOCK, 0)[:n].repeat_interleave(BLOCK, 1)[:, :k].double()
    wd = weight.float().double() * sw
    y = qx @ wd.T
    if bias is not None:
        y = y + bias.double().view(1, -1)
    return y.to(torch.bfloat16)
