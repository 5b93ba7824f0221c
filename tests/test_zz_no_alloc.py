"""The no-allocation GEMM entry point, called through the C ABI.

bfp8_gemm_block128_noalloc is for callers that cannot give the library a workspace because they
cannot allocate device memory where they make the call (a server whose memory pools were sized at
start-up and are closed during decode steps; host code running where CUDA allocation calls are not
allowed).  Its scratch is a fixed array inside the library, shared by every call on the device, so
this test makes two calls in a row and checks each against the ordinary entry point, which is given
a caller-allocated workspace.  The file name makes pytest collect it after every other test.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-2          # max |difference| / rms(expected), the GEMM tolerance of tests/test_gpu_gemm.py


def _operands(m, k, n, seed):
    import gaudi_kernels_b200 as gk
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn((n, k), generator=g) * 0.02).cuda()
    bias = torch.randn(n, generator=g).cuda()
    w_codes, w_scales = gk.quantize_block128(w, native_half=True)
    a_codes, a_scales = gk.quantize_act_1x128(x, native_half=True)      # scales: [M, G] view of [G, M] storage
    return a_codes, a_scales, w_codes, w_scales, bias


@pytest.mark.parametrize("m,k,n,out_dtype", [(8, 1024, 4096, torch.float32), (32, 4096, 14336, torch.bfloat16),
                                             (1, 512, 384, torch.float32)])
def test_noalloc_entry_point_matches_workspace_entry_point(m, k, n, out_dtype):
    from gaudi_kernels_b200 import _lib
    lib = _lib.load()
    a_codes, a_scales, w_codes, w_scales, bias = _operands(m, k, n, seed=m + n)
    sa = a_scales.t().contiguous() if not (m == 1 or a_scales.stride(0) == 1) else a_scales   # group-major storage
    ldsa = m
    code = _lib.OUT_BF16 if out_dtype == torch.bfloat16 else _lib.OUT_F32
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    # ordinary entry point, with a zero-initialised workspace allocated by the caller
    ws_bytes = lib.bfp8_gemm_block128_workspace_bytes(m, n, k)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device="cuda")
    want = torch.empty((m, n), dtype=out_dtype, device="cuda")
    rc = lib.bfp8_gemm_block128(a_codes.data_ptr(), k, sa.data_ptr(), ldsa, w_codes.data_ptr(), k, w_scales.data_ptr(),
                                bias.data_ptr(), want.data_ptr(), code, n, m, n, k, ws.data_ptr(), ws_bytes,
                                status.data_ptr(), stream)
    assert rc == 0
    torch.cuda.synchronize()
    rms = float(want.double().pow(2).mean().sqrt())

    # the entry point under test: no workspace argument, two calls back to back into separate outputs
    outs = [torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda") for _ in range(2)]
    for out in outs:
        rc = lib.bfp8_gemm_block128_noalloc(a_codes.data_ptr(), k, sa.data_ptr(), ldsa, w_codes.data_ptr(), k,
                                            w_scales.data_ptr(), bias.data_ptr(), out.data_ptr(), code, n, m, n, k,
                                            status.data_ptr(), stream)
        assert rc == 0
    # the same schedule through the ordinary interface (weight-streaming form, at most 160 CTAs - the split the
    # built-in scratch is sized for): the no-allocation call must reproduce it bit for bit
    same = torch.empty((m, n), dtype=out_dtype, device="cuda")
    rc = lib.bfp8_gemm_block128_ex(a_codes.data_ptr(), k, sa.data_ptr(), ldsa, w_codes.data_ptr(), k, w_scales.data_ptr(),
                                   bias.data_ptr(), same.data_ptr(), code, n, m, n, k, ws.data_ptr(), ws_bytes,
                                   status.data_ptr(), stream, 2, 160, 0)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for out in outs:
        assert bool(torch.isfinite(out.float()).all())
        err = float((out.double() - want.double()).abs().max())
        assert err / rms <= TOL, err / rms
        assert torch.equal(out, same)


def test_noalloc_entry_point_rejects_sizes_beyond_its_scratch():
    from gaudi_kernels_b200 import _lib
    lib = _lib.load()
    a = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = a.data_ptr()
    # 33 rows: one more than the fixed scratch allows - refused before anything is launched
    rc = lib.bfp8_gemm_block128_noalloc(p, 128, p, 33, p, 128, p, None, p, _lib.OUT_F32, 128, 33, 128, 128, st.data_ptr(), None)
    assert rc == -7
    assert b"scratch" in lib.bfp8_error_string(rc)
    # more 128-row weight tiles than there are counters
    rc = lib.bfp8_gemm_block128_noalloc(p, 128, p, 1, p, 128, p, None, p, _lib.OUT_F32, 1 << 22, 1, (1 << 21) + 129, 128,
                                        st.data_ptr(), None)
    assert rc == -7
