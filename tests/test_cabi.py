"""Host-only checks of the C-ABI library: it builds, loads without a GPU, and exports what the header declares."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from gaudi_kernels_b200 import _lib, build
    build.build()
    return _lib.load()


def _declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(bfp8_\w+)\s*\(", text))
    return names


def test_header_symbols_are_exported(lib):
    from gaudi_kernels_b200 import _lib
    declared = _declared_symbols()
    assert len(declared) >= 9
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), name
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_version_and_error_strings(lib):
    assert lib.bfp8_version() >= 1
    assert lib.bfp8_error_string(0) == b"ok"
    for code in range(-7, 0):
        assert lib.bfp8_error_string(code) not in (b"ok", b"unknown error")
    assert lib.bfp8_gemm_block128_workspace_bytes(8192, 14336, 4096) >= 0


def test_weights_at_rest_switch_is_host_state(lib):
    # a process-wide flag: returns the previous setting, off by default, touches no device
    prev = lib.bfp8_set_weights_at_rest(0)
    try:
        assert lib.bfp8_set_weights_at_rest(1) == 0
        assert lib.bfp8_set_weights_at_rest(5) == 1           # any non-zero value means "at rest"
        assert lib.bfp8_set_weights_at_rest(0) == 1
        assert lib.bfp8_set_weights_at_rest(0) == 0
    finally:
        lib.bfp8_set_weights_at_rest(prev)


def test_host_side_argument_checks_launch_nothing(lib):
    # all of these are rejected before any CUDA call, so they are safe without a device
    assert lib.bfp8_reencode_half(None, None, 16, None, None, 0, None, None, None) == -1
    one = ctypes.c_uint64(0)
    p = ctypes.addressof(one)
    assert lib.bfp8_reencode_half(p, p, 0, None, None, 0, p, p, None) == -3
    assert lib.bfp8_quant_block128_f32(p, 0, 4, 4, p, 4, p, 0, None) == -3
    assert lib.bfp8_quant_act_1x128_bf16(p, 1, 128, 64, p, 128, p, 1, 1, 0, None, None) == -3
    assert lib.bfp8_decode_block128(p, 4, 4, 4, p, p, 7, 4, None) == -3
    # GEMM: misaligned leading dimension, then bad shape
    a = 4096
    assert lib.bfp8_gemm_block128(a, 130, a, 8, a, 136, a, None, a, 1, 16, 8, 16, 130, None, 0, a, None) == -2
    assert lib.bfp8_gemm_block128(a, 128, a, 8, a, 128, a, None, a, 1, 16, 0, 16, 128, None, 0, a, None) == -3
    assert lib.bfp8_gemm_block128(None, 128, a, 8, a, 128, a, None, a, 1, 16, 8, 16, 128, None, 0, a, None) == -1


def test_python_wrappers_validate_like_the_reference():
    import torch
    import gaudi_kernels_b200 as gk
    w = torch.tensor([[0x08, 0x10, 0x78], [0x03, 0x7E, 0x80]], dtype=torch.uint8).view(torch.float8_e4m3fn)
    s = torch.tensor([[0.25, 0.5]], dtype=torch.float32)
    with pytest.raises(ValueError):
        gk.reencode_e4m3fn_half(w.t(), s)                       # non-contiguous
    with pytest.raises(ValueError):
        gk.reencode_e4m3fn_half(w, s.to(torch.float64))         # wrong scale dtype
    with pytest.raises(ValueError):
        gk.reencode_e4m3fn_half(w.view(torch.uint8), s)         # wrong weight dtype
    x = torch.zeros((1, 256), dtype=torch.bfloat16)
    wt = torch.zeros((128, 256), dtype=torch.uint8).view(torch.float8_e4m3fn)
    with pytest.raises(ValueError, match="scale grid"):
        gk.reference(x, wt, torch.ones((1, 1)))
    with pytest.raises(ValueError):
        gk.reference(x.float(), wt, torch.ones((1, 2)))


def test_no_silent_fallback_without_a_gpu():
    import torch
    import gaudi_kernels_b200 as gk
    from gaudi_kernels_b200._lib import Bfp8Error
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    w = torch.zeros(16, dtype=torch.uint8).view(torch.float8_e4m3fn)
    with pytest.raises(Bfp8Error):
        gk.reencode_e4m3fn_half(w, torch.ones(1))


def test_rank_sum_contract_without_gpu():
    """World sizes outside 2..8 are refused before any CUDA call (generic_dense_glue.cpp:576), as are null
    pointers and empty slices; the CPU restatement applies the same rule."""
    import ctypes
    from gaudi_kernels_b200 import _lib
    from oracle import rank_sum_ref
    lib = _lib.load()
    buf = (ctypes.c_float * 64)()
    for world in (1, 9, 0, -3):
        assert lib.bfp8_rank_sum(buf, buf, 8, world, _lib.OUT_F32, None) == -6          # BFP8_ERR_UNSUPPORTED
        with pytest.raises(ValueError):
            rank_sum_ref.check_contract(8 * max(world, 1), 8, world)
    assert lib.bfp8_rank_sum(None, buf, 8, 4, _lib.OUT_F32, None) == -1
    assert lib.bfp8_rank_sum(buf, buf, 0, 4, _lib.OUT_F32, None) == -3          # BFP8_ERR_SHAPE
    assert lib.bfp8_rank_sum(buf, buf, 8, 4, 7, None) == -3
    with pytest.raises(ValueError):
        rank_sum_ref.check_contract(8192, 4096, 4)                # mismatched gathered size (contract test :584)
    rank_sum_ref.check_contract(16384, 4096, 4)


def test_rank_sum_restatement_known_answers():
    import torch
    from oracle import rank_sum_ref
    # fp32: (1e8 + 1) - 1e8 = 0 in rank order 0,1,2 but 1 in the order 0,2,1
    x = torch.tensor([1e8, 1.0, -1e8], dtype=torch.float32)
    assert float(rank_sum_ref.rank_sum(x, 3)[0]) == 0.0
    # bf16: the sum is formed in fp32 and rounded once: 1 + 2^-8 + 2^-8 = 1 + 2^-7 is representable,
    # whereas rounding after each addition would have stayed at 1
    y = torch.tensor([1.0, 2.0 ** -8, 2.0 ** -8], dtype=torch.bfloat16)
    assert float(rank_sum_ref.rank_sum(y, 3)[0]) == 1.0 + 2.0 ** -7
    two = torch.tensor([1.5, -0.25, 2.0, 4.0], dtype=torch.float32)
    assert rank_sum_ref.rank_sum(two, 2).tolist() == [3.5, 3.75]


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs on host cores only and prints one JSON line with the agreed keys."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "0",
                          "--cpu-rows", "2", "--cpu-budget-s", "1"], capture_output=True, text=True, timeout=300, cwd=root)
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "block_fp8_gemm_tflops" and line["unit"] == "TFLOP/s"
    assert line["steps"] == 2 and line["n_gpus"] == 1 and line["higher_is_better"] is True and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0 and "prefill_up" in line["config"]["workload"]
