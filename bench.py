#!/usr/bin/env python
"""Benchmark of the block-FP8 GEMM hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one pass of the block-scaled E4M3 GEMM over one batch of synthetic, already-quantized
operands resident in HBM.  Workloads (synthetic data with the shapes and value distributions of the
FFN projections the path is quoted on; A ~ N(0,1) bf16 quantized 1x128, W ~ N(0,0.02) quantized
128x128 and re-encoded to half-range E4M3):

    prefill_up    M=8192  K=4096  N=14336   (default on 1 GPU: the configuration the target is quoted on)
    prefill_down  M=8192  K=14336 N=4096
    prefill_up_quarter  M=2048 K=4096 N=14336  (small case for profiler captures)
    prefill_up_token_channel  M=8192 K=4096 N=14336 with one scale per token and per output channel
    codec         fp32 [8192, 8192]: the HBM-bound quantize / re-encode / decode kernels, GB/s per kernel
    ffn70b        M=16384 K=8192  N=28672   (default on 2+ GPUs: W split on N over the ranks, A replicated;
                                             total work fixed, so scaling is "strong")

With N > 1 the script expects to be started by torch.distributed.run with one rank per GPU.  Ranks
never exchange data inside the timed step (the output is left column-sharded); the bf16 all-gather a
caller would add when it needs the full output is timed separately and reported under "gather".

--impl reference times the reference's own CPU algorithm for this path (the oracle restatement of
block_fp8_oracle.reference, torch CPU with all host threads) on a bounded row sample of the same
workload, on rank 0 only.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "prefill_up": (8192, 4096, 14336),
    "prefill_down": (8192, 14336, 4096),
    "ffn70b": (16384, 8192, 28672),
    "prefill_up_quarter": (2048, 4096, 14336),     # same kernel and K/N, a quarter of the rows: the size used for ncu captures
    "prefill_up_token_channel": (8192, 4096, 14336),   # same shape, per-token / per-channel scales (no per-block promotion)
    "ffn70b_slice_quarter": (4096, 8192, 3584),    # a quarter of the rows of one rank's slice at 8 GPUs (M=16384, N=28672 / 8): ncu captures
    "decode_m64": (64, 4096, 14336),               # the decode bucket's largest M: the weight-streaming schedule, HBM-bound
    "ffn70b_down": (16384, 28672, 8192),           # row-parallel: W split on K, rank-order sum over peer memory (N > 1 only)
    "codec": (8192, 8192, 0),                      # the elementwise codec configuration, fp32 [8192, 8192] (no GEMM)
}
METRIC = "block_fp8_gemm_tflops"
UNIT = "TFLOP/s"
L2_FLUSH_BYTES = 256 << 20


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=None, help="steps of the host-buffer leg (default: min(steps, 5))")
    ap.add_argument("--cpu-rows", type=int, default=32, help="activation rows of the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-budget-s", type=float, default=120.0,
                    help="host time the --impl reference run aims to take in all (sizes its per-step sample)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the codec, decode-bucket and checkpoint-stream figures of the N=1 line (short profiler runs)")
    return ap.parse_args()


def make_config(workload, m, k, n, world):
    """The `config` object of the JSON line; both arms (ours and --impl reference) print the same one."""
    return {"workload": "%s M=%d K=%d N=%d" % (workload, m, k, n),
            "sharding": "W rows (N) split over %d ranks, A replicated, output left sharded" % world if world > 1 else "single GPU",
            "l2": "256 MiB buffer rewritten between timed steps (L2 is 126 MB); each step timed with its own CUDA events",
            "timed": "GEMM on pre-quantized operands resident in HBM"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        # FP8 dense tensor throughput is twice the bf16 rate on this part; the measured bf16 burst
        # figure (a cuBLAS GEMM timed alone, as this kernel is) is doubled to get the denominator.
        return 2.0 * float(d["bf16_tflops"]), "2 x measured bf16 cuBLAS burst (MEASURED_PEAKS.json)", float(d["hbm_gbs"])
    return 2.0 * 1590.0, "2 x fallback bf16 figure (no MEASURED_PEAKS.json)", 6650.0


def profiled_traffic(workload):
    """DRAM bytes per launch of the GEMM kernel from the committed ncu summary, if one exists."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get(workload)
    return None


def sliced_traffic(workload, m, k, n_local):
    """DRAM bytes per launch of one rank's slice of the multi-GPU shape, scaled from the ncu capture of a quarter of
    its rows (profiles/gemm_block128_dram_traffic.md): A and the output grow with M, the W slice does not.  Only the
    8-GPU slice (N / 8 columns) was captured; other slices give None."""
    q = profiled_traffic("ffn70b_slice_quarter")
    qm, qk, qn = WORKLOADS["ffn70b_slice_quarter"]
    if workload != "ffn70b" or q is None or (k, n_local) != (qk, qn):
        return None
    w_bytes = qk * qn
    return int((q - w_bytes) * (m / qm) + w_bytes)


class ClockSampler:
    """SM clock and throttle reasons sampled through NVML (what nvidia-smi reads) while the timed region runs.

    Read-only queries from a background thread every ~2 ms; nothing on the GPU is changed.
    """

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples = []
        self.reason_bits = 0
        self.sm_max = None
        self.power = []
        self._stop = False
        self._thread = None

    def _resolve_handle(self, nv):
        # CUDA_VISIBLE_DEVICES may renumber devices: match the CUDA device by its PCI bus id
        import torch
        try:
            bus = torch.cuda.get_device_properties(self.gpu_index).pci_bus_id
            dom = torch.cuda.get_device_properties(self.gpu_index).pci_domain_id
            dev = torch.cuda.get_device_properties(self.gpu_index).pci_device_id
            return nv.nvmlDeviceGetHandleByPciBusId(("%08x:%02x:%02x.0" % (dom, bus, dev)).encode())
        except Exception:
            return nv.nvmlDeviceGetHandleByIndex(self.gpu_index)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = self._resolve_handle(nv)
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        except Exception:
            return
        import threading

        def loop():
            while not self._stop:
                try:
                    self.samples.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                    self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                    self.power.append(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)
                except Exception:
                    pass
                time.sleep(0.002)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=2)
        out = {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": len(self.samples)}
        if self.samples:
            out["sm_mhz"] = statistics.median(self.samples)
            out["sm_min_mhz"] = min(self.samples)
            out["power_w_max"] = max(self.power) if self.power else None
            out["reasons"] = sorted(name for bit, name in self.REASONS.items() if self.reason_bits & bit)
            out["how"] = "NVML, sampled every ~2 ms during the timed region only"
        return out


def bench_codec(torch, lib, device, steps, warmup):
    """HBM-bound codec kernels on the fp32 [8192, 8192] configuration (N(0, 0.02) with 0.1 % outliers at 50x).

    Inputs rotate over several buffer sets (together far larger than the 126 MB L2); launches are timed in
    back-to-back batches with CUDA events, and the figure is algorithmic bytes / median time per launch.
    """
    r = c = 8192
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=device).manual_seed(2)
    status = torch.zeros(4, dtype=torch.int32, device=device)
    nb = 4
    src = []
    for _ in range(nb):
        t = torch.randn((r, c), generator=g, device=device) * 0.02
        mask = torch.rand((r, c), generator=g, device=device) < 1e-3
        src.append(torch.where(mask, t * 50, t))
        del t, mask
    ocp = [torch.empty((r, c), dtype=torch.uint8, device=device) for _ in range(nb)]
    half = [torch.empty((r, c), dtype=torch.uint8, device=device) for _ in range(nb)]
    sc = [torch.empty((r // 128, c // 128), dtype=torch.float32, device=device) for _ in range(nb)]
    sc2 = [torch.empty_like(sc[0]) for _ in range(nb)]
    xs = [src[i].view(-1)[: r * c // 2].view(r, c // 2).to(torch.bfloat16) for i in range(nb)]   # bf16 [8192, 4096]
    xs = xs + [x.clone() for x in xs]
    xc = [torch.empty((r, c // 2), dtype=torch.uint8, device=device) for _ in range(len(xs))]
    xsc = torch.empty((c // 2 // 128, r), dtype=torch.float32, device=device)

    def timed(fns):
        """Median time of one launch, measured over batches of back-to-back launches.

        A launch lasts 20-80 us, so a batch of 2 x len(fns) launches (each on a different buffer set) sits between
        one CUDA-event pair: the host's launch latency then hides behind the previous kernel instead of being timed.
        """
        n = len(fns)
        batch = 2 * n
        for i in range(max(warmup, 3) * n):
            fns[i % n]()
        torch.cuda.synchronize()
        ts = []
        for _ in range(max(steps, 8)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(batch):
                rc = fns[i % n]()
                assert rc == 0, rc
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / batch)
        return statistics.median(ts)

    out = {}
    ms = timed([(lambda i=i: lib.bfp8_quant_block128_f32(src[i].data_ptr(), r, c, c, ocp[i].data_ptr(), c, sc[i].data_ptr(), 0, stream))
                for i in range(nb)])
    ms_h = timed([(lambda i=i: lib.bfp8_quant_block128_f32(src[i].data_ptr(), r, c, c, half[i].data_ptr(), c, sc2[i].data_ptr(), 1, stream))
                  for i in range(nb)])
    out["quantize_block128_halve"] = {"ms": ms_h, "bytes": r * c * 5, "gbs": r * c * 5 / ms_h / 1e6}
    out["quantize_block128_ocp"] = {"ms": ms, "bytes": r * c * 5, "gbs": r * c * 5 / ms / 1e6}
    ms = timed([(lambda i=i: lib.bfp8_reencode_half(ocp[i].data_ptr(), half[(i + 1) % nb].data_ptr(), r * c, sc[i].data_ptr(),
                                                    sc2[i].data_ptr(), sc[i].numel(), status.data_ptr(), status.data_ptr() + 8, stream))
                for i in range(nb)])
    out["reencode_half"] = {"ms": ms, "bytes": r * c * 2, "gbs": r * c * 2 / ms / 1e6}
    ms = timed([(lambda i=i: lib.bfp8_decode_block128(half[i].data_ptr(), r, c, c, sc2[i].data_ptr(), src[i].data_ptr(), 0, c, stream))
                for i in range(nb)])
    out["decode_f32"] = {"ms": ms, "bytes": r * c * 5, "gbs": r * c * 5 / ms / 1e6}
    m, k = r, c // 2
    ms = timed([(lambda i=i: lib.bfp8_quant_act_1x128_bf16(xs[i].data_ptr(), m, k, k, xc[i].data_ptr(), k, xsc.data_ptr(), 1, m, 1,
                                                           None, stream)) for i in range(len(xs))])
    nbytes = m * k * 3 + (k // 128) * m * 4
    out["quantize_act_1x128"] = {"ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "shape": "bf16 [8192, 4096]"}
    # per-token quantizer (one scale per row): 2 B in + 1 B out per element + 4 B per row
    tsc = torch.empty(m, dtype=torch.float32, device=device)
    ms = timed([(lambda i=i: lib.bfp8_quant_act_token_bf16(xs[i].data_ptr(), m, k, k, xc[i].data_ptr(), k, tsc.data_ptr(), 1,
                                                           None, stream)) for i in range(len(xs))])
    nbytes = m * k * 3 + m * 4
    out["quantize_act_token"] = {"ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "shape": "bf16 [8192, 4096]"}
    # the two activation quantizers on the activation of the multi-GPU workload (a launch of [8192, 4096] lasts about
    # 20 us, of which the ramp at either end is a visible part)
    del xs, xc
    m, k = WORKLOADS["ffn70b"][0], WORKLOADS["ffn70b"][1]
    xs = [torch.randn((m, k), generator=g, device=device).to(torch.bfloat16) for _ in range(3)]
    xc = [torch.empty((m, k), dtype=torch.uint8, device=device) for _ in range(3)]
    xsc = torch.empty((k // 128, m), dtype=torch.float32, device=device)
    tsc = torch.empty(m, dtype=torch.float32, device=device)
    ms = timed([(lambda i=i: lib.bfp8_quant_act_1x128_bf16(xs[i].data_ptr(), m, k, k, xc[i].data_ptr(), k, xsc.data_ptr(), 1, m, 1,
                                                           None, stream)) for i in range(len(xs))])
    nbytes = m * k * 3 + (k // 128) * m * 4
    out["quantize_act_1x128_16384x8192"] = {"ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "shape": "bf16 [16384, 8192]"}
    ms = timed([(lambda i=i: lib.bfp8_quant_act_token_bf16(xs[i].data_ptr(), m, k, k, xc[i].data_ptr(), k, tsc.data_ptr(), 1,
                                                           None, stream)) for i in range(len(xs))])
    nbytes = m * k * 3 + m * 4
    out["quantize_act_token_16384x8192"] = {"ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "shape": "bf16 [16384, 8192]"}
    # the re-encode on the 70B-class weight [28672, 8192] (235 MB each way; the [8192, 8192] launch above lasts 25 us)
    del xs, xc
    wn, wk = WORKLOADS["ffn70b"][2], WORKLOADS["ffn70b"][1]
    wsrc = [torch.randint(0, 0x7f, (wn, wk), generator=g, device=device, dtype=torch.uint8) for _ in range(3)]
    wdst = [torch.empty((wn, wk), dtype=torch.uint8, device=device) for _ in range(3)]
    wsc = torch.rand((wn // 128, wk // 128), generator=g, device=device) + 0.01
    wsc2 = torch.empty_like(wsc)
    ms = timed([(lambda i=i: lib.bfp8_reencode_half(wsrc[i].data_ptr(), wdst[i].data_ptr(), wn * wk, wsc.data_ptr(), wsc2.data_ptr(),
                                                    wsc.numel(), status.data_ptr(), status.data_ptr() + 8, stream)) for i in range(3)])
    out["reencode_half_28672x8192"] = {"ms": ms, "bytes": wn * wk * 2, "gbs": wn * wk * 2 / ms / 1e6, "shape": "e4m3 [28672, 8192]"}
    return out


def bench_decode_bucket(torch, lib, device, k=4096, n=14336, reps=20, rounds=8, ms=(1, 8, 32, 64)):
    """Small-M GEMM (the decode bucket) at one weight shape: HBM-bound on the 58.7 MB of weight codes.

    The weight fits in L2, so launches rotate over four weight copies; `reps` launches are captured in one CUDA
    graph (host launch latency is longer than the kernel) and the graph is timed with CUDA events.
    """
    g = torch.Generator(device=device).manual_seed(3)
    ws_codes = [torch.randint(0, 0x77, (n, k), generator=g, device=device, dtype=torch.uint8) for _ in range(4)]
    w_scales = torch.rand((n // 128, k // 128), generator=g, device=device) * 1e-3
    status = torch.zeros(4, dtype=torch.int32, device=device)
    out = {}
    for m in ms:
        a_codes = torch.randint(0, 0x77, (m, k), generator=g, device=device, dtype=torch.uint8)
        a_scales = torch.rand((k // 128, m), generator=g, device=device)
        y = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        ws_bytes = lib.bfp8_gemm_block128_workspace_bytes(m, n, k)
        ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=device)

        def launch(count):
            stream = torch.cuda.current_stream().cuda_stream
            for i in range(count):
                rc = lib.bfp8_gemm_block128(a_codes.data_ptr(), k, a_scales.data_ptr(), m, ws_codes[i % 4].data_ptr(), k,
                                            w_scales.data_ptr(), None, y.data_ptr(), 1, n, m, n, k, ws.data_ptr(), ws_bytes,
                                            status.data_ptr() + 8, stream)
                assert rc == 0, rc

        launch(4)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            launch(reps)
        ts = []
        for _ in range(rounds):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / reps)
        us = statistics.median(ts) * 1e3
        nbytes = n * k + 4 * (n // 128) * (k // 128) + m * k + 4 * m * (k // 128) + 2 * m * n
        out["M=%d" % m] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "tflops": round(2.0 * m * n * k / us / 1e6, 1),
                           "bytes": nbytes}
    return out


def bench_decode_ffn(torch, lib, device, hidden=4096, inter=14336, reps=10, rounds=8):
    """One FFN of a decode step.  Headline form, four kernels: 1x128 quantize -> gate/up GEMM on the interleaved weight with
    the SwiGLU step in its epilogue (bf16 [M, I]) -> 1x128 quantize -> down GEMM [M, hidden].  Beside it the five-kernel form
    without the fused epilogue: gate GEMM and up GEMM into the two halves of one [M, 2 I] buffer (separate launches of
    I = 14336 columns each: 112 tiles, one CTA per tile) -> silu_and_mul fused into the 1x128 quantizer -> down GEMM.
    Captured `reps` times in a CUDA graph over two rotating sets of weights (352 MB, larger than L2); all kernels are
    launched with programmatic stream serialization, so each one's launch and set-up overlap the tail of the one
    before.  HBM-bound on the 176 MB of weight codes per FFN."""
    g = torch.Generator(device=device).manual_seed(9)
    sets = []
    for _ in range(2):
        sets.append((torch.randint(0, 0x77, (2 * inter, hidden), generator=g, device=device, dtype=torch.uint8),
                     torch.rand((2 * inter // 128, hidden // 128), generator=g, device=device) * 1e-3,
                     torch.randint(0, 0x77, (hidden, inter), generator=g, device=device, dtype=torch.uint8),
                     torch.rand((hidden // 128, inter // 128), generator=g, device=device) * 1e-3))
    status = torch.zeros(4, dtype=torch.int32, device=device)
    out = {}
    for m in (1, 8, 64):
        x = torch.randn((m, hidden), generator=g, device=device).to(torch.bfloat16)
        a1 = torch.empty((m, hidden), dtype=torch.uint8, device=device)
        s1 = torch.empty((hidden // 128, m), dtype=torch.float32, device=device)
        gu = torch.empty((m, 2 * inter), dtype=torch.bfloat16, device=device)
        a2 = torch.empty((m, inter), dtype=torch.uint8, device=device)
        s2 = torch.empty((inter // 128, m), dtype=torch.float32, device=device)
        y = torch.empty((m, hidden), dtype=torch.bfloat16, device=device)
        ws_bytes = max(lib.bfp8_gemm_block128_workspace_bytes(m, 2 * inter, hidden),
                       lib.bfp8_gemm_block128_workspace_bytes(m, hidden, inter))
        ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=device)
        sp = status.data_ptr() + 8

        def ffn(count):
            st = torch.cuda.current_stream().cuda_stream
            for i in range(count):
                wgu, sgu, wd, sd = sets[i % 2]
                rcs = (lib.bfp8_quant_act_1x128_bf16(x.data_ptr(), m, hidden, hidden, a1.data_ptr(), hidden, s1.data_ptr(), 1, m, 1, None, st),
                       lib.bfp8_gemm_block128(a1.data_ptr(), hidden, s1.data_ptr(), m, wgu.data_ptr(), hidden, sgu.data_ptr(), None,
                                              gu.data_ptr(), 1, 2 * inter, m, inter, hidden, ws.data_ptr(), ws_bytes, sp, st),
                       lib.bfp8_gemm_block128(a1.data_ptr(), hidden, s1.data_ptr(), m, wgu.data_ptr() + inter * hidden, hidden,
                                              sgu.data_ptr() + 4 * (inter // 128) * (hidden // 128), None,
                                              gu.data_ptr() + 2 * inter, 1, 2 * inter, m, inter, hidden, ws.data_ptr(), ws_bytes, sp, st),
                       lib.bfp8_silu_quant_act_1x128_bf16(gu.data_ptr(), m, inter, 2 * inter, a2.data_ptr(), inter, s2.data_ptr(),
                                                          1, m, 1, None, st),
                       lib.bfp8_gemm_block128(a2.data_ptr(), inter, s2.data_ptr(), m, wd.data_ptr(), inter, sd.data_ptr(), None,
                                              y.data_ptr(), 1, hidden, m, hidden, inter, ws.data_ptr(), ws_bytes, sp, st))
                assert rcs == (0, 0, 0, 0, 0), rcs

        h = torch.empty((m, inter), dtype=torch.bfloat16, device=device)

        def ffn_fused(count):
            # the same step on the interleaved gate/up weight (the copy the prefill kernel reads): one GEMM whose
            # epilogue applies SwiGLU, then the plain 1x128 quantizer - four kernels, no [M, 2 I] round trip
            st = torch.cuda.current_stream().cuda_stream
            for i in range(count):
                wgu, sgu, wd, sd = sets[i % 2]
                rcs = (lib.bfp8_quant_act_1x128_bf16(x.data_ptr(), m, hidden, hidden, a1.data_ptr(), hidden, s1.data_ptr(), 1, m, 1, None, st),
                       lib.bfp8_gemm_block128_swiglu(a1.data_ptr(), hidden, s1.data_ptr(), m, wgu.data_ptr(), hidden, sgu.data_ptr(), None,
                                                     h.data_ptr(), inter, m, inter, hidden, ws.data_ptr(), ws_bytes, sp, st),
                       lib.bfp8_quant_act_1x128_bf16(h.data_ptr(), m, inter, inter, a2.data_ptr(), inter, s2.data_ptr(), 1, m, 1, None, st),
                       lib.bfp8_gemm_block128(a2.data_ptr(), inter, s2.data_ptr(), m, wd.data_ptr(), inter, sd.data_ptr(), None,
                                              y.data_ptr(), 1, hidden, m, hidden, inter, ws.data_ptr(), ws_bytes, sp, st))
                assert rcs == (0, 0, 0, 0), rcs

        def timed_graph(fn):
            fn(2)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn(reps)
            ts = []
            for _ in range(rounds):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graph.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) / reps)
            return statistics.median(ts) * 1e3

        us = timed_graph(ffn)
        us_fused = timed_graph(ffn_fused)
        nbytes = 3 * inter * hidden                                  # weight codes; everything else is below 1 %
        out["M=%d" % m] = {"us": round(us_fused, 2), "weight_gbs": round(nbytes / us_fused / 1e3, 1), "kernels": 4,
                           "us_unfused_5_kernels": round(us, 2)}
    assert int(status.cpu()[2]) == 0
    return out


def bench_checkpoint_stream(torch, device, tensors=12, n=8192, k=8192):
    """Load-time pipeline: `tensors` pinned host weights of n x k codes streamed to the GPU and re-encoded.

    Bound by the host-to-device link; the re-encode of tensor t runs under the copy of tensor t + 1.
    """
    from gaudi_kernels_b200.checkpoint import stream_checkpoint
    g = torch.Generator().manual_seed(5)
    w = torch.randint(0, 0x77, (n, k), generator=g, dtype=torch.uint8).pin_memory()
    s = torch.rand((n // 128, k // 128), generator=g) + 0.01
    entries = [("w%d" % i, w, s) for i in range(tensors)]
    stream_checkpoint(entries[:2], device=device)                       # warm-up: streams, staging, first launches
    nbytes = tensors * (n * k + s.numel() * 4)
    rates = []
    for _ in range(2):      # the first pass pays cudaMalloc for the resident tensors, the second reuses their blocks
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = stream_checkpoint(entries, device=device)
        torch.cuda.synchronize()
        rates.append(round(nbytes / (time.perf_counter() - t0) / 1e9, 1))
        del out
    return {"gbs": rates[1], "gbs_first_pass_with_cudamalloc": rates[0], "bytes": nbytes, "tensors": tensors,
            "source": "pinned host memory"}


def measure_row_parallel(torch, dist, gk, device, m, k, n, world, rank, steps, warmup, sample_clocks=True):
    """K-sharded down projection: every rank multiplies its K slice and the partials are added in rank order.

    Operands are drawn directly as codes (the quantizers are timed elsewhere).  A step is the fused form:
    GEMM whose epilogue stores its bf16 tiles into the owning GPU's memory, barrier, local rank-order sum, barrier.
    The unfused form (local partial, then a sum kernel that reads the peers' rows) and the GEMM alone are timed
    beside it.  Returns a dict; every rank must call it.
    """
    from gaudi_kernels_b200 import row_parallel as rp
    k0, k1 = rp.k_shard_bounds(k, world, rank)
    kl = k1 - k0
    g = torch.Generator(device=device).manual_seed(17 + rank)
    a_codes = torch.randint(0, 0x77, (m, kl), generator=g, device=device, dtype=torch.uint8)
    a_scales = torch.rand((kl // 128, m), generator=g, device=device).t()
    w_codes = torch.randint(0, 0x77, (n, kl), generator=g, device=device, dtype=torch.uint8)
    w_scales = torch.rand((n // 128, kl // 128), generator=g, device=device) * 1e-3
    ex = rp.PeerExchange(m * n * 2)
    r0, r1 = rp.row_bounds(m, world, rank)
    out = torch.empty((r1 - r0, n), dtype=torch.bfloat16, device=device)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    fused = rp.push_supported(m, n, world)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            flush.zero_()
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        ms = []
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            ms.append((e0, e1))
        dist.barrier()
        torch.cuda.synchronize()
        total = torch.tensor([sum(a.elapsed_time(b) for a, b in ms)], dtype=torch.float64, device=device)
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
        return float(total.item()) / steps

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", 0)))
    if rank == 0 and sample_clocks:
        sampler.start()
    ms = timed(lambda: rp.gemm_k_sharded(a_codes, a_scales, w_codes, w_scales, ex, out=out, fused=fused), steps, warmup)
    clocks = sampler.stop() if (rank == 0 and sample_clocks) else None
    ms_unfused = timed(lambda: rp.gemm_k_sharded(a_codes, a_scales, w_codes, w_scales, ex, out=out, fused=False),
                       min(steps, 10), 3)
    local = ex.partial(m, n, torch.bfloat16)
    ms_gemm = timed(lambda: gk.gemm_block_fp8(a_codes, a_scales, w_codes, w_scales, out=local, check=False, status=ex.status),
                    min(steps, 10), 3)
    timed_out = ex.timed_out()
    ex.close()
    return {"ms": ms, "unfused_ms": ms_unfused, "gemm_only_ms": ms_gemm, "fused": fused, "timed_out": timed_out,
            "clocks": clocks, "nvlink_bytes_into_each_gpu": (world - 1) * (m // world) * n * 2}


def row_parallel_parity(torch, dist, gk, device, world, rank):
    """A small K-sharded product on all ranks: fused == unfused bit for bit, and both against the CPU oracle
    (per-rank partials by oracle.block_fp8_ref, then the restated rank-order sum of oracle.rank_sum_ref)."""
    from gaudi_kernels_b200 import row_parallel as rp
    from oracle import block_fp8_ref, fp8_codec_ref, rank_sum_ref
    m, k, n = 128 * world * 2, 256 * world, 512
    g = torch.Generator().manual_seed(4321)                                  # every rank builds the same problem
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    codes_np, scales_np = fp8_codec_ref.quantize_block128((torch.randn((n, k), generator=g) * 0.02).numpy())
    codes, s = torch.from_numpy(codes_np).view(torch.float8_e4m3fn), torch.from_numpy(scales_np)
    k0, k1 = rp.k_shard_bounds(k, world, rank)
    w_dev, s_dev = gk.prepare_weight(codes.to(device), s.to(device), native_half=True)
    w_loc, s_loc = rp.shard_weight_k(w_dev, s_dev, world, rank)
    a_codes, a_scales = gk.quantize_act_1x128(x[:, k0:k1].contiguous().to(device), native_half=True)
    ex = rp.PeerExchange(m * n * 2)
    fused = rp.gemm_k_sharded(a_codes, a_scales, w_loc, s_loc, ex, fused=True).clone()
    unfused = rp.gemm_k_sharded(a_codes, a_scales, w_loc, s_loc, ex, fused=False).clone()
    torch.cuda.synchronize()
    timed_out = ex.timed_out()
    ex.close()
    r0, r1 = rp.row_bounds(m, world, rank)
    parts64, parts = [], []
    for r in range(world):
        a0, a1 = rp.k_shard_bounds(k, world, r)
        y64, ybf = block_fp8_ref.reference_rows(x[r0:r1, a0:a1].contiguous(), codes[:, a0:a1].contiguous(),
                                                s[:, a0 // 128:(a1 + 127) // 128].contiguous(), native_half=True)
        parts64.append(y64)
        parts.append(ybf)
    want = rank_sum_ref.rank_sum(torch.stack(parts).reshape(-1).contiguous(), world).view(r1 - r0, n)
    total64 = sum(parts64)
    rms = float(total64.pow(2).mean().sqrt())
    got = fused.cpu()
    # the gate of tests/test_gpu_row_parallel.py: the GEMM tolerance per rank plus one bf16 step per rounding
    bound = 1e-2 * rms * world + (world + 1) * 2.0 ** -7 * float(total64.abs().max())
    gate_ok = (float((got.double() - total64).abs().max()) <= bound and float((got.double() - want.double()).abs().max()) <= bound)
    stats = torch.tensor([float((got.double() - total64).abs().max()) / rms,
                          float((got.double() - want.double()).abs().max()) / rms,
                          0.0 if torch.equal(fused, unfused) else 1.0, 1.0 if timed_out else 0.0, 0.0 if gate_ok else 1.0],
                         dtype=torch.float64, device=device)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    st = stats.tolist()
    return {"shape": "M=%d K=%d N=%d" % (m, k, n), "max_err_over_rms_vs_fp64": st[0],
            "max_diff_over_rms_vs_oracle_bf16_partials_and_rank_sum": st[1], "fused_equals_unfused_bitwise": st[2] == 0.0,
            "barrier_wait_expired": st[3] != 0.0, "within_gate_on_every_rank": st[4] == 0.0,
            "gate": "1e-2 of the RMS per rank plus one bf16 step per rounding (W + 1 roundings), as tests/test_gpu_row_parallel.py"}


def run_row_parallel(args, torch, dist, gk, device, workload, m, k, n, world, rank):
    if world < 2:
        raise SystemExit("ffn70b_down is a multi-GPU workload: start it with torch.distributed.run and --gpus N >= 2")
    res = measure_row_parallel(torch, dist, gk, device, m, k, n, world, rank, args.steps, max(args.warmup, 3))
    parity = row_parallel_parity(torch, dist, gk, device, world, rank)
    ms, fused = res["ms"], res["fused"]
    if rank == 0:
        flops = 2.0 * m * k * n
        peak_tflops, peak_how, _ = measured_peaks()
        line = {"metric": METRIC, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32, bf16 partials, fp32 rank-order sum (bf16 out)",
                "data": "synthetic",
                "config": {"workload": "%s M=%d K=%d N=%d" % (workload, m, k, n),
                           "sharding": "W and A split on K over %d ranks; rank r keeps output rows [r M / W, (r + 1) M / W)" % world,
                           "form": "fused: tiles stored to the owning GPU by the GEMM epilogue" if fused else "unfused",
                           "l2": "256 MiB buffer rewritten between timed steps",
                           "timed": "GEMM + inter-GPU barrier + rank-order sum + barrier, operands resident in HBM"},
                "roofline": {"bound": "tensor", "achieved": flops / world / (ms * 1e-3) / 1e12, "peak": peak_tflops,
                             "unit": "TFLOP/s", "frac": flops / world / (ms * 1e-3) / 1e12 / peak_tflops,
                             "peak_source": peak_how + " - of measured", "traffic": None,
                             "kernel": "gemm_block128_kernel<bf16 out> (push mode) + rank_sum_kernel"},
                "compare": {"unfused_ms_per_step": res["unfused_ms"], "local_gemm_only_ms": res["gemm_only_ms"],
                            "nvlink_bytes_into_each_gpu": res["nvlink_bytes_into_each_gpu"]},
                "row_parallel_parity": parity,
                "clocks": res["clocks"], "gpu_launches": 4 * args.steps, "barrier_wait_expired": res["timed_out"]}
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def make_problem(torch, gk, m, k, n_local, n_offset, n_total, device, seed=0):
    """Synthetic operands: bf16 activations and an fp32 weight slice, quantized on the GPU by the library."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((m, k), generator=g, dtype=torch.float32).to(torch.bfloat16)
    # the weight slice of this rank is generated from a per-slice seed so no rank materialises the full matrix
    gw = torch.Generator(device=device).manual_seed(1000 + n_offset)
    w = torch.randn((n_local, k), generator=gw, device=device, dtype=torch.float32) * 0.02
    w_ocp, s_ocp = gk.quantize_block128(w)
    del w
    return x, w_ocp, s_ocp


def run_reference(args, workload, m, k, n, world, rank):
    """The reference's CPU algorithm (oracle restatement) on a bounded sample; rank 0 only."""
    if rank != 0:
        return
    import torch
    from oracle import block_fp8_ref, fp8_codec_ref
    import numpy as np
    # launchers such as torch.distributed.run pin OMP_NUM_THREADS to 1; the CPU arm uses every host core
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    rng = np.random.default_rng(0)
    wf = torch.randn((n, k), generator=torch.Generator().manual_seed(1)) * 0.02
    codes, scales = fp8_codec_ref.quantize_block128(wf.numpy())
    del wf
    w = torch.from_numpy(codes).view(torch.float8_e4m3fn)
    s = torch.from_numpy(scales)
    x_all = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).to(torch.bfloat16)

    def one(rows):
        t0 = time.perf_counter()
        block_fp8_ref.reference(x_all[:rows], w, s, native_half=True)
        return time.perf_counter() - t0

    # Size the per-step sample so that the whole run (warm-up and timed steps alike) takes about two minutes: a
    # call costs a fixed part (weight preparation) plus a per-row part, both measured here on two small samples.
    r_small, r_big = max(1, args.cpu_rows), min(m, 8 * max(1, args.cpu_rows))
    t_small, t_big = one(r_small), one(r_big)
    per_row = max((t_big - t_small) / max(r_big - r_small, 1), 1e-9)
    fixed = max(t_small - per_row * r_small, 0.0)
    warmup = max(args.warmup, 0)
    budget = args.cpu_budget_s / max(args.steps + warmup, 1)
    rows = int(min(m, max(r_small, (budget - fixed) / per_row)))
    rows = max(r_small, rows // 32 * 32 if rows >= 32 else rows)
    flops = 2.0 * rows * k * n
    times = []
    for i in range(warmup + args.steps):
        dt = one(rows)
        if i >= warmup:
            times.append(dt)
    per_step = sum(times) / len(times)
    value = flops / per_step / 1e12
    sample = ("%d of the workload's %d activation rows per step (full K and N, weight preparation included); "
              "the sample is sized so that warm-up and timed steps together take about %.0f s" % (rows, m, args.cpu_budget_s))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
        "steps": len(times), "warmup": warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f64 (exact E4M3 products)",
        "data": "synthetic",
        "config": make_config(workload, m, k, n, world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    if args.gpus > 1 and world == 1:
        raise SystemExit("start multi-GPU runs with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    workload = args.workload or ("prefill_up" if world == 1 else "ffn70b")
    m, k, n = WORKLOADS[workload]

    if args.impl == "reference":
        run_reference(args, workload, m, k, n, world, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    import gaudi_kernels_b200 as gk
    from gaudi_kernels_b200 import _lib
    lib = _lib.load()

    if workload == "ffn70b_down":
        run_row_parallel(args, torch, dist, gk, device, workload, m, k, n, world, rank)
        return

    if workload == "decode_m64":
        # the decode bucket: a launch is shorter than the host's launch path, so launches are timed inside a CUDA
        # graph (20 per replay, four rotating weight copies: W always comes from DRAM), not one event pair each
        if rank == 0:
            rounds = max(args.steps, 8)
            res = bench_decode_bucket(torch, lib, device, k, n, reps=20, rounds=rounds, ms=(m,))["M=%d" % m]
            _, _, hbm_gbs = measured_peaks()
            line = {"metric": METRIC, "value": res["tflops"], "unit": UNIT, "n_gpus": 1, "steps": 20 * rounds,
                    "warmup": 4, "ms_per_step": res["us"] * 1e-3, "higher_is_better": True, "scaling": "weak",
                    "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 (bf16 out)", "data": "synthetic",
                    "config": {"workload": "%s M=%d K=%d N=%d" % (workload, m, k, n),
                               "l2": "launches rotate over four copies of W (235 MB, larger than L2)",
                               "timed": "CUDA graph of 20 launches per replay, median over replays"},
                    "roofline": {"bound": "hbm", "achieved": res["gbs"], "peak": hbm_gbs, "unit": "GB/s",
                                 "frac": res["gbs"] / hbm_gbs, "peak_source": "MEASURED_PEAKS.json hbm_gbs - of measured",
                                 "traffic": profiled_traffic(workload), "kernel": "gemm_smallm_kernel<MP=64>",
                                 "algorithmic_bytes": res["bytes"]},
                    "gpu_launches": 20 * rounds}
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    if workload == "codec":
        # codec kernels only (single GPU; every rank would do identical work)
        if rank == 0:
            res = bench_codec(torch, lib, device, args.steps, args.warmup)
            _, _, hbm_gbs = measured_peaks()
            main_k = res["quantize_block128_halve"]
            line = {"metric": "codec_hbm_gbs", "value": main_k["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": max(args.steps, 8),
                    "warmup": max(args.warmup, 3), "ms_per_step": main_k["ms"], "higher_is_better": True, "scaling": "weak",
                    "vs_baseline": None, "dtype": "f32 -> e4m3 (u8)", "data": "synthetic",
                    "config": {"workload": "codec fp32 [8192, 8192]: quantize 128x128 + halve (5 B/elem)",
                               "l2": "inputs rotate over 4 buffer sets (1 GiB), far larger than L2"},
                    "roofline": {"bound": "hbm", "achieved": main_k["gbs"], "peak": hbm_gbs, "unit": "GB/s",
                                 "frac": main_k["gbs"] / hbm_gbs, "peak_source": "MEASURED_PEAKS.json hbm_gbs - of measured",
                                 "traffic": None, "kernel": "quant_block128_kernel"},
                    "kernels": res, "gpu_launches": 5 * 8 * max(args.steps, 8)}
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    if n % (128 * world) != 0:
        raise SystemExit("N must split into 128-aligned slices")
    n_local = n // world
    n_offset = rank * n_local
    x, w_ocp, s_ocp = make_problem(torch, gk, m, k, n_local, n_offset, n, device)
    token_channel = workload.endswith("_token_channel")
    if token_channel:
        # per-channel weight scales: the block-quantized codes are kept, one scale per output channel is drawn
        w_codes = gk.prepare_weight(w_ocp, s_ocp, native_half=True)[0]
        w_scales = torch.rand(n_local, device=device) * 1e-3 + 1e-4
        a_codes, a_scales = gk.quantize_act_token(x.to(device), native_half=True)
        args.no_e2e = True
        args.no_cpu_baseline = True
    else:
        w_codes, w_scales = gk.prepare_weight(w_ocp, s_ocp, native_half=True)
        a_codes, a_scales = gk.quantize_act_1x128(x.to(device), native_half=True)
    out = torch.empty((m, n_local), dtype=torch.bfloat16, device=device)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    flops_total = 2.0 * m * k * n                     # whole job, all ranks

    def step():
        if token_channel:
            gk.gemm_token_channel_fp8(a_codes, a_scales, w_codes, w_scales, out=out, check=False)
        else:
            gk.gemm_block_fp8(a_codes, a_scales, w_codes, w_scales, out=out, check=False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    t_wall = time.perf_counter()
    for i in range(args.steps):
        flush.zero_()                                  # evict operands and output from L2 between timed steps
        starts[i].record()
        step()
        stops[i].record()
    barrier()
    t_wall = time.perf_counter() - t_wall
    clocks = sampler.stop() if rank == 0 else None
    step_ms = [a.elapsed_time(b) for a, b in zip(starts, stops)]
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    ms_per_step = total_ms / args.steps
    value = flops_total / (ms_per_step * 1e-3) / 1e12
    status_timeout = False

    # ---- optional: all-gather of the column-sharded bf16 output (outside the timed step)
    gather = None
    if world > 1:
        full = torch.empty((world * m, n_local), dtype=torch.bfloat16, device=device)
        for _ in range(2):
            dist.all_gather_into_tensor(full, out)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        reps = 5
        for _ in range(reps):
            dist.all_gather_into_tensor(full, out)
        e1.record()
        barrier()
        g_ms = torch.tensor([e0.elapsed_time(e1) / reps], dtype=torch.float64, device=device)
        dist.all_reduce(g_ms, op=dist.ReduceOp.MAX)
        gather = {"ms": float(g_ms.item()), "bytes_into_each_gpu": (world - 1) * m * n_local * 2,
                  "layout": "[world, M, N/world] bf16"}
        del full

    # ---- end to end through the reference-facing call with host buffers
    e2e = None
    if not args.no_e2e:
        e2e_steps = args.e2e_steps or min(args.steps, 5)
        wh = w_ocp.cpu().pin_memory()
        sh = s_ocp.cpu().pin_memory()
        yh = torch.empty((m, n_local), dtype=torch.bfloat16).pin_memory()
        if world == 1:
            xh = x.pin_memory()
            call = lambda: gk.reference(xh, wh, sh, native_half=True, out=yh)   # returns after the result is on the host
            call_name = ("gaudi_kernels_b200.reference(x, weight, scales, native_half=True) on pinned host tensors: "
                         "H2D, re-encode, 1x128 quantize, GEMM, D2H")
            launches = 1 + 2 * (1 if m < 2048 else min(8, m // 1024))
        else:
            from gaudi_kernels_b200 import sharded
            rows = m // world
            xh = x[rank * rows:(rank + 1) * rows].contiguous().pin_memory()      # this rank uploads only its rows
            call = lambda: sharded.reference_sharded(xh, wh, sh, native_half=True, out=yh)
            call_name = ("gaudi_kernels_b200.sharded.reference_sharded(x rows of this rank, weight slice, scales slice) on "
                         "pinned host tensors: H2D, re-encode, 1x128 quantize of M / W rows, all-gather of codes and scales "
                         "(NCCL), GEMM on the rank's columns, D2H of its [M, N / W] slice")
            launches = 2 + max(1, min(8, m // 2048))
        for _ in range(2):
            call()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            call()
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e_s = float(dt.item()) / e2e_steps
        h2d = xh.numel() * 2 + wh.numel() + sh.numel() * 4
        d2h = yh.numel() * 2 + 16
        e2e = {"value": flops_total / e2e_s / 1e12, "unit": UNIT, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "call": call_name,
               "gpu_launches_per_step": launches,
               "bound": "host link of each GPU: %.1f GB/s to the host, %.1f GB/s from it per rank" % (d2h / e2e_s / 1e9, h2d / e2e_s / 1e9)}
        if world > 1:
            e2e["nccl_bytes_into_each_gpu_per_step"] = (world - 1) * (m // world) * (k + 4 * (k // 128))
            e2e["bytes_are_per_rank"] = True

    # ---- N > 1: parity of rank 0's slice, the same problem on one GPU (strong-scaling reference), row-parallel path
    multi = {}
    if world > 1 and not args.no_extras:
        def guarded(key, fn):
            try:
                multi[key] = fn()
            except Exception as e:  # noqa: BLE001 - a side figure never takes the headline down
                multi[key + "_error"] = repr(e)[:300]

        def strong():
            # the unsharded M x K x N product on rank 0's GPU alone, same kernel, same timing rules
            if rank != 0:
                return None
            gg = torch.Generator(device=device).manual_seed(77)
            wf = torch.randint(0, 0x77, (n, k), generator=gg, device=device, dtype=torch.uint8)
            sf = torch.rand((n // 128, k // 128), generator=gg, device=device) * 1e-3
            of = torch.empty((m, n), dtype=torch.bfloat16, device=device)
            ts = []
            for i in range(2 + 5):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                gk.gemm_block_fp8(a_codes, a_scales, wf, sf, out=of, check=False)
                e1.record()
                torch.cuda.synchronize()
                if i >= 2:
                    ts.append(e0.elapsed_time(e1))
            t1 = sum(ts) / len(ts)
            return {"t1_ms": t1, "tN_ms": ms_per_step, "efficiency": t1 / (world * ms_per_step),
                    "how": "t1 = the unsharded M=%d K=%d N=%d product on rank 0's GPU alone in this run (5 steps, L2 flushed); "
                           "efficiency = t1 / (N * tN)" % (m, k, n)}

        def parity():
            if rank != 0:
                return None
            from oracle import block_fp8_ref
            torch.set_num_threads(max(1, os.cpu_count() or 1))
            rows = 32
            yb = block_fp8_ref.reference(x[:rows].contiguous(), w_ocp.cpu(), s_ocp.cpu(), native_half=True)
            got = out[:rows].cpu()
            return {"rows": rows, "columns": "rank 0's slice [0, %d)" % n_local,
                    "max_abs_diff_bf16": (got.double() - yb.double()).abs().max().item(),
                    "rms": float(yb.double().pow(2).mean().sqrt()), "mismatching_elements": int((got != yb).sum())}

        guarded("strong_scaling", strong)
        guarded("parity_sample", parity)
        barrier()
        guarded("row_parallel_parity", lambda: row_parallel_parity(torch, dist, gk, device, world, rank))
        dm, dk, dn = WORKLOADS["ffn70b_down"]
        guarded("ffn70b_down", lambda: measure_row_parallel(torch, dist, gk, device, dm, dk, dn, world, rank, 10, 3,
                                                             sample_clocks=False))
        if "ffn70b_down" in multi:
            r = multi["ffn70b_down"]
            r.pop("clocks", None)
            r["workload"] = "ffn70b_down M=%d K=%d N=%d, W and A split on K" % (dm, dk, dn)
            r["tflops_fused"] = 2.0 * dm * dk * dn / (r["ms"] * 1e-3) / 1e12

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak_tflops, peak_how, hbm_gbs = measured_peaks()
    # the kernel timed is one GEMM launch per step on this rank
    launch_flops = 2.0 * m * k * n_local
    achieved = launch_flops / (statistics.median(step_ms) * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 (bf16 out)",
        "data": "synthetic",
        "config": make_config(workload, m, k, n, world),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tflops, "unit": "TFLOP/s",
                     "frac": achieved / peak_tflops, "peak_source": peak_how + " - of measured",
                     "frac_of_nominal_4500": achieved / 4500.0,
                     "traffic": profiled_traffic(workload) if world == 1 else sliced_traffic(workload, m, k, n_local),
                     "kernel": "gemm_channel_kernel<bf16 out>" if token_channel else "gemm_block128_kernel<bf16 out>",
                     "launch_ms_median": statistics.median(step_ms)},
        "clocks": clocks,
        "gpu_launches": args.steps,
        "wall_s_timed_region": t_wall,
    }
    if world == 1 and not token_channel and not args.no_extras:
        # side figures of the N=1 line; a failure in one of them is reported in the line, not raised, so that the
        # headline measurement above is never lost to it
        def extra(key, fn):
            try:
                fn()
            except Exception as e:  # noqa: BLE001
                line[key + "_error"] = repr(e)[:300]

        def extra_codec():
            codec = bench_codec(torch, lib, device, 8, 3)
            line["codec_hbm_gbs"] = {k: round(v["gbs"], 1) for k, v in codec.items()}
            line["codec_hbm_frac_of_measured"] = {k: round(v["gbs"] / hbm_gbs, 3) for k, v in codec.items()}
            line["codec_hbm_frac_of_nominal_8000"] = {k: round(v["gbs"] / 8000.0, 3) for k, v in codec.items()}

        # The decode figures are taken as a serving process runs them: the weights were written long before the
        # timed launches, so the library is told that they are at rest (each GEMM may then ask for its first weight
        # tiles while the kernel before it drains).  "us_weights_not_at_rest" is the M=1 figure without that promise.
        def extra_decode():
            for dk, dn in ((4096, 14336), (14336, 4096)):
                prev = lib.bfp8_set_weights_at_rest(1)
                try:
                    decode = bench_decode_bucket(torch, lib, device, dk, dn)
                    lib.bfp8_set_weights_at_rest(0)
                    plain = bench_decode_bucket(torch, lib, device, dk, dn, ms=(1,))
                finally:
                    lib.bfp8_set_weights_at_rest(prev)
                for v in decode.values():
                    v["hbm_frac_of_measured"] = round(v["gbs"] / hbm_gbs, 3)
                decode["M=1"]["us_weights_not_at_rest"] = plain["M=1"]["us"]
                decode["weights_at_rest"] = True
                line["decode_bucket_k%d_n%d" % (dk, dn)] = decode

        def extra_ffn():
            prev = lib.bfp8_set_weights_at_rest(1)
            try:
                ffn = bench_decode_ffn(torch, lib, device)
            finally:
                lib.bfp8_set_weights_at_rest(prev)
            for v in ffn.values():
                v["hbm_frac_of_measured"] = round(v["weight_gbs"] / hbm_gbs, 3)
            ffn["weights_at_rest"] = True
            line["decode_ffn_hidden4096_inter14336"] = ffn

        def extra_checkpoint():
            line["checkpoint_stream_h2d_reencode"] = bench_checkpoint_stream(torch, device)

        def extra_ffn70b():
            # the multi-GPU workload, unsharded, on this one GPU: the t1 of the strong-scaling curve
            fm, fk, fn = WORKLOADS["ffn70b"]
            gg = torch.Generator(device=device).manual_seed(77)
            af = torch.randint(0, 0x77, (fm, fk), generator=gg, device=device, dtype=torch.uint8)
            asf = torch.rand((fk // 128, fm), generator=gg, device=device).t()
            wf = torch.randint(0, 0x77, (fn, fk), generator=gg, device=device, dtype=torch.uint8)
            sf = torch.rand((fn // 128, fk // 128), generator=gg, device=device) * 1e-3
            of = torch.empty((fm, fn), dtype=torch.bfloat16, device=device)
            ts = []
            for i in range(2 + 5):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                gk.gemm_block_fp8(af, asf, wf, sf, out=of, check=False)
                e1.record()
                torch.cuda.synchronize()
                if i >= 2:
                    ts.append(e0.elapsed_time(e1))
            t1 = sum(ts) / len(ts)
            line["ffn70b_1gpu"] = {"ms": t1, "tflops": 2.0 * fm * fk * fn / (t1 * 1e-3) / 1e12,
                                   "workload": "ffn70b M=%d K=%d N=%d unsharded (5 steps, L2 flushed)" % (fm, fk, fn)}

        extra("ffn70b_1gpu", extra_ffn70b)
        extra("codec_hbm_gbs", extra_codec)
        extra("decode_bucket", extra_decode)
        extra("decode_ffn", extra_ffn)
        extra("checkpoint_stream", extra_checkpoint)
    for key, val in multi.items():
        if val is not None:
            line[key] = val
    if gather is not None:
        line["gather"] = gather
    if e2e is not None:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        from oracle import block_fp8_ref
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        rows = max(1, args.cpu_rows)
        xs = x[:rows].contiguous()
        wc, sc = w_ocp.cpu(), s_ocp.cpu()
        t0 = time.perf_counter()
        yb = block_fp8_ref.reference(xs, wc, sc, native_half=True)
        dt = time.perf_counter() - t0
        for _ in range(3):
            if dt >= 5.0 or rows >= m:
                break
            # the sample was short (a small sample's time is mostly weight preparation): grow it towards about
            # ten seconds of host work, so that the per-row cost dominates the figure
            rows = int(min(m, max(2 * rows, rows * 10.0 / dt))) // 32 * 32 or rows
            xs = x[:rows].contiguous()
            t0 = time.perf_counter()
            yb = block_fp8_ref.reference(xs, wc, sc, native_half=True)
            dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 2.0 * rows * k * n / dt / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
                                "kind": "port", "seconds": dt,
                                "sample": "first %d of %d activation rows, full K and N, weight preparation included" % (rows, m)}
        # the sample doubles as a parity spot check of the benchmarked output
        got = out[:rows].cpu()
        diff = (got.double() - yb.double()).abs().max().item()
        line["parity_sample"] = {"rows": rows, "max_abs_diff_bf16": diff,
                                 "rms": float(yb.double().pow(2).mean().sqrt())}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
