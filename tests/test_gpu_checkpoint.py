"""GPU test of the load-time pipeline: streamed re-encode of many host tensors equals the per-tensor codec."""

import numpy as np
import pytest
import torch

from oracle import fp8_codec_ref, swiglu_ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gk():
    import gaudi_kernels_b200 as g
    from gaudi_kernels_b200 import _lib
    _lib.load()
    return g


def _tensor(n, k, seed, pinned=False):
    rng = np.random.default_rng(seed)
    w = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
    w[(w & 0x7f) == 0x7f] ^= 0x01                                  # no NaN codes
    s = rng.random(((n + 127) // 128, (k + 127) // 128), dtype=np.float32) + np.float32(0.01)
    wt = torch.from_numpy(w).view(torch.float8_e4m3fn)
    if pinned:
        wt = wt.view(torch.uint8).pin_memory().view(torch.float8_e4m3fn)
    return wt, torch.from_numpy(s)


def test_streamed_checkpoint_equals_per_tensor_codec(gk):
    from gaudi_kernels_b200.checkpoint import stream_checkpoint
    shapes = [(256, 384), (1024, 4096), (130, 200), (4096, 1024), (512, 512), (1, 7), (2048, 2048)]
    tensors = {"layer%d.w" % i: _tensor(n, k, seed=i, pinned=(i % 3 == 0)) for i, (n, k) in enumerate(shapes)}
    consumed = []

    def entries():                                                 # a generator: tensors are pulled one at a time
        for name, (w, s) in tensors.items():
            consumed.append(name)
            yield name, w, s

    got = stream_checkpoint(entries(), native_half=True, staging_bytes=1 << 16)     # staging buffers must grow
    assert consumed == list(tensors) and list(got) == list(tensors)
    for name, (w, s) in tensors.items():
        codes, scales, rounded = got[name]
        want_codes, want_scales, want_rounded = fp8_codec_ref.reencode_e4m3fn_half(w.view(torch.uint8).numpy(), s.numpy())
        assert codes.dtype == torch.float8_e4m3fn and codes.device.type == "cuda"
        assert np.array_equal(codes.view(torch.uint8).cpu().numpy(), want_codes), name
        assert np.array_equal(scales.cpu().numpy(), want_scales), name
        assert rounded == want_rounded, name
    # OCP codes kept as they are
    plain = stream_checkpoint(((n, w, s) for n, (w, s) in tensors.items()), native_half=False)
    for name, (w, s) in tensors.items():
        assert torch.equal(plain[name][0].view(torch.uint8).cpu(), w.view(torch.uint8))
        assert torch.equal(plain[name][1].cpu(), s) and plain[name][2] == 0
    # ... and still checked: a NaN code or a negative / non-finite scale is rejected, naming the tensor
    name, (w, s) = next(iter(tensors.items()))
    bad_w = w.view(torch.uint8).clone()
    bad_w[-1, -1] = 0xFF
    with pytest.raises(ValueError, match="nonfinite"):
        stream_checkpoint([(name, bad_w.view(torch.float8_e4m3fn), s)], native_half=False)
    for bad in (-1.0, float("inf"), float("nan")):
        bad_s = s.clone()
        bad_s.view(-1)[0] = bad
        with pytest.raises(ValueError, match=name):
            stream_checkpoint([(name, w, bad_s)], native_half=False)


def test_streamed_checkpoint_swiglu_entry_and_errors(gk):
    from gaudi_kernels_b200.checkpoint import stream_checkpoint
    w, s = _tensor(512, 1000, seed=9)                              # I = 256, K padded to 1008 for the interleave
    other_w, other_s = _tensor(256, 256, seed=10)
    got = stream_checkpoint([("mlp.gate_up", w, s), ("mlp.down", other_w, other_s)], swiglu=["mlp.gate_up"])
    codes = got["mlp.gate_up"][0].view(torch.uint8).cpu().numpy()
    half, _, _ = fp8_codec_ref.reencode_e4m3fn_half(w.view(torch.uint8).numpy(), s.numpy())
    assert codes.shape == (512, 1008) and not codes[:, 1000:].any()
    assert np.array_equal(codes[:, :1000], swiglu_ref.interleave_gate_up(half))
    want_il, want_s = gk.prepare_weight_swiglu(w.cuda(), s.cuda(), native_half=True)
    assert torch.equal(got["mlp.gate_up"][0].view(torch.uint8), want_il.view(torch.uint8))
    assert got["mlp.down"][0].shape == (256, 256)

    bad_w = w.clone().view(torch.uint8)
    bad_w[3, 5] = 0x7f
    with pytest.raises(ValueError, match="second.*nonfinite"):
        stream_checkpoint([("first", other_w, other_s), ("second", bad_w.view(torch.float8_e4m3fn), s)])
    bad_s = s.clone()
    bad_s[0, 0] = -1.0
    with pytest.raises(ValueError, match="neg.*scales"):
        stream_checkpoint([("neg", w, bad_s)])
    with pytest.raises(ValueError, match="grid"):
        stream_checkpoint([("shape", w, s[:1])])
    with pytest.raises(ValueError, match="duplicate"):
        stream_checkpoint([("a", other_w, other_s), ("a", other_w, other_s)])
    with pytest.raises(ValueError, match="multiple of 128"):
        stream_checkpoint([("odd", *_tensor(384, 128, seed=3))], swiglu=["odd"])
    assert stream_checkpoint([]) == {}
