#!/usr/bin/env python
"""o_proj alone over the token range of the named GQA configuration (1 ... 512 tokens) for every rank's K-slice
(cp = 1, 2, 4, 8 -> K = 8192 ... 1024, hidden 8192), against torch.nn.functional.linear (cuBLAS), one GPU.

    python benchmarks/oproj_tokens_bench.py [--iters 20]

Rotating weight buffers larger than L2, CUDA events, >= 3 warm-ups; one JSON line per point.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import torch  # noqa: E402

from benchmarks.kernel_bench import measured_peaks, time_rotating  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", default="1,8,32,64,128,256,384,512")
    args = ap.parse_args()
    os.environ.setdefault("HELIX_A2A_ENABLE_PDL", "1")
    from helix_a2a_b200.ops.oproj import oproj, prepack_weight, check_compute_status
    hbm, _, src = measured_peaks()
    hidden = 8192
    for cp in (1, 2, 4, 8):
        K = 8192 // cp
        nl = max(2, (512 * 1024 * 1024) // (hidden * K * 2))
        ws = [(torch.randn(hidden, K, device="cuda") * 0.02).bfloat16() for _ in range(nl)]
        wp = [prepack_weight(w) for w in ws]
        for T in [int(t) for t in args.tokens.split(",")]:
            x = torch.randn(T, K, device="cuda").bfloat16()
            us = time_rotating([(lambda l=l: oproj(x, wp[l])) for l in range(nl)], args.iters)
            us_ref = time_rotating([(lambda l=l: torch.nn.functional.linear(x, ws[l])) for l in range(nl)], args.iters)
            nbytes = hidden * K * 2 + T * K * 2 + T * hidden * 2
            print(json.dumps({"kernel": "oproj (packed weights)", "cp": cp, "K": K, "tokens": T, "us": us,
                              "torch_linear_us": us_ref, "frac_of_%s_hbm" % src: nbytes / us / 1e3 / hbm,
                              "tflops": 2 * T * K * hidden / us / 1e6}), flush=True)
            check_compute_status(x)
        del ws, wp


if __name__ == "__main__":
    main()
