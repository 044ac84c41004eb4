"""Operator micro-benchmark: times single kernels of the evaluation path through the C ABI's
stand-alone operator entry points, on the matrix shapes of the BT4-class network.

    python -m lc0_b200.opbench gemm [--batch 1024] [--precision fp16] [--reps 5] [--only NAME]

Prints one line per shape with the CUDA-event time and achieved TFLOP/s.  Small enough to run under
`ncu -k regex:gemm_tc --set full` (use --batch 64..256 and --reps 1 for a capture).
"""
import argparse
import sys

import numpy as np


def gemm_shapes(batch):
    t = batch * 64
    return [("qkv", t, 3072, 1024), ("proj", t, 1024, 1024), ("ffn1", t, 1536, 1024), ("ffn2", t, 1024, 1536),
            ("smolgen_compress", t, 32, 1024), ("smolgen_dense1", batch, 256, 2048),
            ("smolgen_dense2", batch, 8192, 256), ("smolgen_global", batch * 32, 4096, 256),
            ("embedding", t, 1024, 624), ("policy_emb", t, 1024, 1024),
            # one tile per CTA and one k-block: what a launch costs besides its work
            ("fixed_cost", 128, 64, 64), ("fixed_cost_pair", 512, 9728, 64)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm"])
    ap.add_argument("--batch", type=int, default=1024)
    ap.add_argument("--precision", default="fp16")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--only", default="")
    ap.add_argument("--fma", action="store_true", help="time the FMA kernel instead of the tensor-core kernel")
    args = ap.parse_args()
    import torch
    from . import _lib
    lib = _lib.load()
    prec = _lib.PRECISIONS[args.precision]
    dt = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[prec]
    for name, M, N, K in gemm_shapes(args.batch):
        if args.only and args.only != name:
            continue
        A = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
        W = (torch.randn(N, K, device="cuda") * K ** -0.5).to(dt)
        b = torch.randn(N, device="cuda")
        C = torch.empty(M, N, dtype=dt, device="cuda")
        times = []
        for r in range(args.reps + 1):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(lib.b200_op_gemm(A.data_ptr(), W.data_ptr(), b.data_ptr(), C.data_ptr(), M, N, K, 3, prec,
                                        0 if args.fma else 1, None))
            e1.record()
            torch.cuda.synchronize()
            if r > 0 or args.reps == 0:
                times.append(e0.elapsed_time(e1))
        ms = float(np.median(times)) if times else float("nan")
        print("%-18s M=%-7d N=%-5d K=%-5d %8.3f ms  %8.1f TFLOP/s" % (name, M, N, K, ms, 2.0 * M * N * K / ms / 1e9),
              flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
