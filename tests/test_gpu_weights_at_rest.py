"""bfp8_set_weights_at_rest: the decode-bucket GEMMs request their weight before the previous kernel has finished.

Only the weight may be read early.  The checks chain quantizer -> GEMM launches in which every GEMM's activation
codes and scales are produced by the kernel right before it (in the same buffers, with different inputs per step),
so a kernel that read its activations or scales before the wait would pick up the previous step's values; results
must be bit-identical to the same chain with the switch off.
"""
import pytest
import torch

import gaudi_kernels_b200 as gk
from gaudi_kernels_b200 import _lib

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture
def at_rest():
    prev = gk.set_weights_at_rest(True)
    try:
        yield
    finally:
        gk.set_weights_at_rest(prev)


def _weights(n, k, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    codes = torch.randint(0, 0x77, (n, k), generator=g, device=DEV, dtype=torch.uint8)
    codes |= (torch.randint(0, 2, (n, k), generator=g, device=DEV, dtype=torch.uint8) << 7)
    scales = torch.rand((n // 128, k // 128), generator=g, device=DEV) * 1e-2 + 1e-4
    return codes, scales


def _chain(xs, w_codes, w_scales, swiglu):
    """quantize -> GEMM for every x in xs, all launches back to back on one stream, shared activation buffers."""
    lib = _lib.load()
    m, k = xs[0].shape
    n = w_codes.shape[0]
    a = torch.empty((m, k), dtype=torch.uint8, device=DEV)
    sa = torch.empty((k // 128, m), dtype=torch.float32, device=DEV)
    width = n // 2 if swiglu else n
    outs = [torch.empty((m, width), dtype=torch.bfloat16, device=DEV) for _ in xs]
    ws_bytes = lib.bfp8_gemm_block128_workspace_bytes(m, n, k)
    ws = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    for x, y in zip(xs, outs):
        rc = lib.bfp8_quant_act_1x128_bf16(x.data_ptr(), m, k, k, a.data_ptr(), k, sa.data_ptr(), 1, m, 1, None, st)
        assert rc == 0, rc
        if swiglu:
            rc = lib.bfp8_gemm_block128_swiglu(a.data_ptr(), k, sa.data_ptr(), m, w_codes.data_ptr(), k, w_scales.data_ptr(),
                                               None, y.data_ptr(), width, m, width, k, ws.data_ptr(), ws_bytes,
                                               status.data_ptr() + 8, st)
        else:
            rc = lib.bfp8_gemm_block128(a.data_ptr(), k, sa.data_ptr(), m, w_codes.data_ptr(), k, w_scales.data_ptr(), None,
                                        y.data_ptr(), 1, n, m, n, k, ws.data_ptr(), ws_bytes, status.data_ptr() + 8, st)
        assert rc == 0, rc
    torch.cuda.synchronize()
    assert int(status.cpu()[2]) == 0
    return outs


# one CTA per tile (112 tiles); stream-K with partial sums (224 tiles, 16 padded rows); clusters (32 tiles, long K);
# a short K range that does not fill the pipeline
SHAPES = [(1, 4096, 14336), (64, 4096, 14336), (8, 4096, 28672), (32, 14336, 4096), (5, 256, 1024), (128, 1024, 2048)]


@pytest.mark.parametrize("m,k,n", SHAPES)
def test_chain_is_bit_identical_with_weights_at_rest(m, k, n):
    w_codes, w_scales = _weights(n, k, seed=m + n)
    g = torch.Generator(device=DEV).manual_seed(17)
    xs = [(torch.randn((m, k), generator=g, device=DEV) * (0.25 + i)).to(torch.bfloat16) for i in range(6)]
    prev = gk.set_weights_at_rest(False)
    try:
        plain = _chain(xs, w_codes, w_scales, swiglu=False)
        assert gk.set_weights_at_rest(True) is False
        early = _chain(xs, w_codes, w_scales, swiglu=False)
        assert gk.set_weights_at_rest(False) is True
    finally:
        gk.set_weights_at_rest(prev)
    for i, (p, e) in enumerate(zip(plain, early)):
        assert torch.equal(p, e), "step %d differs" % i
    # the steps really differ from one another, so a stale activation would have shown
    assert not torch.equal(plain[0], plain[1])


@pytest.mark.parametrize("m,k,inter", [(1, 4096, 14336), (64, 4096, 14336), (16, 1024, 1024)])
def test_swiglu_chain_is_bit_identical_with_weights_at_rest(m, k, inter, at_rest):
    w_codes, w_scales = _weights(2 * inter, k, seed=m + inter)
    g = torch.Generator(device=DEV).manual_seed(23)
    xs = [(torch.randn((m, k), generator=g, device=DEV) * (0.5 + i)).to(torch.bfloat16) for i in range(4)]
    early = _chain(xs, w_codes, w_scales, swiglu=True)
    gk.set_weights_at_rest(False)
    plain = _chain(xs, w_codes, w_scales, swiglu=True)
    for i, (p, e) in enumerate(zip(plain, early)):
        assert torch.equal(p, e), "step %d differs" % i


def test_graph_replay_with_weights_at_rest(at_rest):
    """The same chain captured in a CUDA graph (programmatic edges between the kernels) and replayed twice."""
    m, k, n = 8, 4096, 14336
    w_codes, w_scales = _weights(n, k, seed=5)
    g = torch.Generator(device=DEV).manual_seed(29)
    xs = [(torch.randn((m, k), generator=g, device=DEV) * (1 + i)).to(torch.bfloat16) for i in range(5)]
    want = _chain(xs, w_codes, w_scales, swiglu=False)
    lib = _lib.load()
    a = torch.empty((m, k), dtype=torch.uint8, device=DEV)
    sa = torch.empty((k // 128, m), dtype=torch.float32, device=DEV)
    outs = [torch.zeros((m, n), dtype=torch.bfloat16, device=DEV) for _ in xs]
    ws_bytes = lib.bfp8_gemm_block128_workspace_bytes(m, n, k)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)

    def enqueue():
        st = torch.cuda.current_stream().cuda_stream
        for x, y in zip(xs, outs):
            assert lib.bfp8_quant_act_1x128_bf16(x.data_ptr(), m, k, k, a.data_ptr(), k, sa.data_ptr(), 1, m, 1, None, st) == 0
            assert lib.bfp8_gemm_block128(a.data_ptr(), k, sa.data_ptr(), m, w_codes.data_ptr(), k, w_scales.data_ptr(), None,
                                          y.data_ptr(), 1, n, m, n, k, ws.data_ptr(), ws_bytes, status.data_ptr() + 8, st) == 0

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        enqueue()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        enqueue()
    for _ in range(2):
        for y in outs:
            y.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for i, (w, y) in enumerate(zip(want, outs)):
            assert torch.equal(w, y), "step %d differs" % i
    assert int(status.cpu()[2]) == 0
