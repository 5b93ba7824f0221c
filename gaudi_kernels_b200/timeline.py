"""In-kernel timeline of the two block-FP8 GEMM kernels (diagnostic; needs a B200).

    python -m gaudi_kernels_b200.build --timeline
    python -m gaudi_kernels_b200.timeline large  [M K N]      # default 8192 4096 14336
    python -m gaudi_kernels_b200.timeline smallm [M K N]      # default 64 4096 14336

Loads libbfp8_timeline.so (the library compiled with -DBFP8_TIMELINE), runs a few launches on seeded random codes and
prints, for one CTA, the SM-clock stamp of every pipeline event of its first 40 units of work (a K block of a
128 x 256 tile, or a 16 KB unit of the weight-streaming schedule), relative to the first stamp, and the medians of
the intervals that bound the kernel.  The stamps cost a few cycles each, so the intervals read a little longer than
in the product build; the order of magnitude and the ranking of the steps are what they are for.
"""

import ctypes
import os
import sys

import numpy as np
import torch

from . import _lib

HERE = os.path.dirname(os.path.abspath(__file__))
EVENTS, UNITS = 8, 40      # kTimelineEvents, kTimelineUnits of csrc/common.cuh

LARGE_EVENTS = ["producer: stage free, copies issued", "issuer: operands landed and buffer handed back",
                "issuer: 4 MMAs + commit issued", "epilogue: first 64 columns in registers",
                "epilogue: buffer handed back", "epilogue: FMAs of the block issued",
                "epilogue: completion of the next block observed"]
SMALLM_EVENTS = ["producer: stage free, copies issued", "issuer: TMEM buffer free", "issuer: operands landed",
                 "issuer: 4 MMAs + 2 commits issued", "epilogue: turns to the unit", "epilogue: accumulator and scales ready",
                 "epilogue: buffer handed back", "scale loader: scale products parked"]


def _load():
    path = os.path.join(HERE, "libbfp8_timeline.so")
    if not os.path.exists(path):
        raise SystemExit("build it first: python -m gaudi_kernels_b200.build --timeline")
    lib = ctypes.CDLL(path)
    for name, (res, args) in _lib.SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    for name in ("bfp8_timeline_read_large", "bfp8_timeline_read_smallm"):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = ctypes.c_int, [ctypes.c_void_p]
    return lib


def _problem(m, k, n, dev):
    g = torch.Generator(device=dev).manual_seed(11)
    a = torch.randint(0, 0x77, (m, k), generator=g, device=dev, dtype=torch.uint8)
    sa = torch.rand((k // 128, m), generator=g, device=dev)
    w = [torch.randint(0, 0x77, (n, k), generator=g, device=dev, dtype=torch.uint8) for _ in range(3)]
    sw = torch.rand((n // 128, k // 128), generator=g, device=dev) * 1e-3
    y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    return a, sa, w, sw, y


def _check(lib, rc):
    if rc != 0:
        raise SystemExit("launch failed: %s (CUDA error %d)" % (lib.bfp8_error_string(rc).decode(), lib.bfp8_last_cuda_error()))


def _stamps(read):
    buf = np.zeros((EVENTS, UNITS), dtype=np.uint32)
    rc = read(buf.ctypes.data)
    if rc != 0:
        raise SystemExit("timeline read failed: %d" % rc)
    return buf.astype(np.int64)


def _print(title, names, t, pairs):
    reached = int((t[1] != 0).sum())
    t0 = int(t[0, 0])
    rel = ((t - t0 + (1 << 31)) & 0xFFFFFFFF) - (1 << 31)       # 32-bit clock: wrap-safe, events before the first stamp negative
    print(title)
    for i, name in enumerate(names):
        print("  [%d] %s" % (i, name))
    print("  unit " + " ".join("%8s" % ("[%d]" % i) for i in range(len(names))))
    for u in range(reached):
        print("  %4d " % u + " ".join("%8d" % int(rel[i, u]) for i in range(len(names))))
    lo, hi = min(8, reached // 4), reached - 4                   # the formulas look up to four units ahead
    print("  medians over units %d..%d (SM cycles):" % (lo, hi - 1))
    for label, fn in pairs:
        vals = [fn(rel, u) for u in range(lo, hi)]
        print("    %-64s %6d" % (label, int(np.median(vals))))


def main(argv):
    kind = argv[0] if argv else "large"
    dims = [int(x) for x in argv[1:4]] if len(argv) >= 4 else None
    dev = torch.device("cuda:0")
    lib = _load()
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    if kind == "large":
        m, k, n = dims or (8192, 4096, 14336)
        a, sa, w, sw, y = _problem(m, k, n, dev)
        for i in range(4):
            rc = lib.bfp8_gemm_block128_ex(a.data_ptr(), k, sa.data_ptr(), m, w[i % 3].data_ptr(), k, sw.data_ptr(), None,
                                           y.data_ptr(), 1, n, m, n, k, None, 0, status.data_ptr() + 8, st, 1, 0, 0)
            _check(lib, rc)
        t = _stamps(lib.bfp8_timeline_read_large)
        _print("large-tile kernel, M=%d K=%d N=%d: K blocks of one CTA" % (m, k, n), LARGE_EVENTS, t, [
            ("K block interval (issuer: operands landed, block to block)", lambda r, u: r[1, u + 1] - r[1, u]),
            ("issuing 4 MMAs + commit", lambda r, u: r[2, u] - r[1, u]),
            ("commit issued -> first 64 columns in registers (MMA time + hand-over)", lambda r, u: r[3, u] - r[2, u]),
            ("first columns in registers -> buffer handed back", lambda r, u: r[4, u] - r[3, u]),
            ("buffer handed back -> MMAs of block u + 2 can be issued", lambda r, u: r[1, u + 2] - r[4, u]),
            ("hand-back -> FMAs of the block issued", lambda r, u: r[5, u] - r[4, u]),
            ("FMAs issued -> completion of the next block observed", lambda r, u: r[6, u] - r[5, u]),
        ])
    elif kind == "smallm":
        m, k, n = dims or (64, 4096, 14336)
        a, sa, w, sw, y = _problem(m, k, n, dev)
        ws_bytes = lib.bfp8_gemm_block128_workspace_bytes(m, n, k)
        ws = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        for i in range(6):
            rc = lib.bfp8_gemm_block128_ex(a.data_ptr(), k, sa.data_ptr(), m, w[i % 3].data_ptr(), k, sw.data_ptr(), None,
                                           y.data_ptr(), 1, n, m, n, k, ws.data_ptr(), ws_bytes, status.data_ptr() + 8, st,
                                           2, 0, 0)
            _check(lib, rc)
        t = _stamps(lib.bfp8_timeline_read_smallm)
        _print("weight-streaming kernel, M=%d K=%d N=%d: 16 KB units of one CTA" % (m, k, n), SMALLM_EVENTS, t, [
            ("unit interval (epilogue: buffer handed back, unit to unit)", lambda r, u: r[6, u + 1] - r[6, u]),
            ("copies issued -> operands landed", lambda r, u: r[2, u] - r[0, u]),
            ("issuing 4 MMAs + 2 commits", lambda r, u: r[3, u] - r[2, u]),
            ("commits issued -> the issuer's next buffer-free check passes (same thread)",
             lambda r, u: (r[1, u + 2] - r[3, u]) if m > 32 else (r[1, u + 4] - r[3, u])),
            ("epilogue: turns to the unit -> accumulator and scales ready", lambda r, u: r[5, u] - r[4, u]),
            ("epilogue: ready -> buffer handed back (TMEM loads)", lambda r, u: r[6, u] - r[5, u]),
            ("epilogue: handed back -> turns to the next unit (FMAs)", lambda r, u: r[4, u + 1] - r[6, u]),
        ])
    else:
        raise SystemExit(__doc__)
    torch.cuda.synchronize()
    assert int(status.cpu()[2]) == 0, "device status %d" % int(status.cpu()[2])


if __name__ == "__main__":
    main(sys.argv[1:])
