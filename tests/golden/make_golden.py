"""Generate golden vectors by running the unmodified reference implementation.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/gaudi-kernels

It imports gaudi_kernels.fp8_codec.reencode_e4m3fn_half and
gaudi_kernels.block_fp8_oracle.reference from <checkout>/python, feeds them the
seeded inputs built by tests/golden/cases.py, and stores inputs and outputs as
.npz files next to this script.  The test-suite reads only the .npz files.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python make_golden.py <path to a checkout of tracycam/gaudi-kernels>")
    ref_root = sys.argv[1]
    sys.path.insert(0, os.path.join(ref_root, "python"))
    from gaudi_kernels.block_fp8_oracle import reference
    from gaudi_kernels.fp8_codec import reencode_e4m3fn_half

    # ---- codec ---------------------------------------------------------------------
    out = {}
    for name, (codes, scales) in cases.codec_cases().items():
        w = torch.from_numpy(codes).view(torch.float8_e4m3fn)
        enc, adj, rounded = reencode_e4m3fn_half(w, torch.from_numpy(scales))
        out[name + ".codes"] = codes
        out[name + ".scales"] = scales
        out[name + ".encoded"] = enc.view(torch.uint8).numpy()
        out[name + ".adjusted"] = adj.numpy()
        out[name + ".rounded"] = np.int64(rounded)
    np.savez_compressed(os.path.join(HERE, "codec.npz"), **out)

    # ---- GEMM: reference() called row by row, as its contract requires --------------
    out = {}
    for name, c in cases.gemm_cases().items():
        x = torch.from_numpy(c["x_bf16_bits"]).view(torch.bfloat16)
        w = torch.from_numpy(c["w_codes"]).view(torch.float8_e4m3fn)
        s = torch.from_numpy(c["w_scales"])
        bias = None if c["bias"] is None else torch.from_numpy(c["bias"])
        for half in (False, True):
            rows = [reference(x[i:i + 1], w, s, native_half=half, bias=bias) for i in range(x.shape[0])]
            y = torch.cat(rows, 0)
            out[f"{name}.y_bits.half{int(half)}"] = y.view(torch.int16).numpy()
        if c["store_inputs"]:
            out[name + ".x_bf16_bits"] = c["x_bf16_bits"]
            out[name + ".w_codes"] = c["w_codes"]
            out[name + ".w_scales"] = c["w_scales"]
            if c["bias"] is not None:
                out[name + ".bias"] = c["bias"]
        out[name + ".input_digest"] = np.frombuffer(cases.digest(c), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "gemm.npz"), **out)
    print("wrote", os.path.join(HERE, "codec.npz"), os.path.join(HERE, "gemm.npz"))


if __name__ == "__main__":
    main()
