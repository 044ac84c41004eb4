"""Operator micro-benchmark: times single kernels of the evaluation path through the C ABI's
stand-alone operator entry points, on the matrix shapes of the BT4-class network.

    python -m lc0_b200.opbench gemm [--batch 1024] [--precision fp16] [--reps 5] [--only NAME]
    python -m lc0_b200.opbench encode [--batch 65536] [--reps 5]     (device-side position encoder)
    python -m lc0_b200.opbench mux [--threads 64] [--request 16] [--config cfg4]   (batch aggregation across threads)
    python -m lc0_b200.opbench multi [--gpus 8] [--batch 1024] [--reps 5]          (one batch over several GPUs)
    python -m lc0_b200.opbench l2scratch [--slice-kb 1024] [--stream-kb 2048] [--iters 40] [--mode 3]

Prints one line per shape with the CUDA-event time and achieved TFLOP/s.  Small enough to run under
`ncu -k regex:gemm_tc --set full` (use --batch 64..256 and --reps 1 for a capture).
"""
import argparse
import ctypes
import sys

import numpy as np


def gemm_shapes(batch):
    t = batch * 64
    return [("qkv", t, 3072, 1024), ("proj", t, 1024, 1024), ("ffn1", t, 1536, 1024), ("ffn2", t, 1024, 1536),
            ("smolgen_compress", t, 32, 1024), ("smolgen_dense1", batch, 256, 2048),
            ("smolgen_dense2", batch, 8192, 256), ("smolgen_global", batch * 32, 4096, 256),
            ("embedding", t, 1024, 624), ("policy_emb", t, 1024, 1024),
            # one tile per CTA and one k-block: what a launch costs besides its work
            ("fixed_cost", 128, 64, 64), ("fixed_cost_pair", 512, 9472, 64)]


def encode_bench(lib, args):
    """Times b200_op_encode_positions on the fixture histories of tests/golden/encoder_golden.npz tiled to --batch
    positions (last 8 boards each), input format 2, fill policy FEN_ONLY."""
    import os
    import torch
    from . import _lib
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    g = np.load(os.path.join(root, "tests", "golden", "encoder_golden.npz"))
    offs = g["offsets"]
    hists = [g["boards"][max(int(offs[i]), int(offs[i + 1]) - 8):int(offs[i + 1])] for i in range(len(offs) - 1)]
    fs = [bool(g["from_start"][i]) and int(offs[i + 1]) - int(offs[i]) <= 8 for i in range(len(offs) - 1)]
    n = args.batch
    order = [i % len(hists) for i in range(n)]
    boards = np.concatenate([hists[i] for i in order])
    offsets = np.concatenate([[0], np.cumsum([len(hists[i]) for i in order])]).astype(np.int32)
    d_boards = torch.from_numpy(boards.view(np.uint8).reshape(-1, 88).copy()).cuda()
    d_offsets = torch.from_numpy(offsets).cuda()
    d_fs = torch.from_numpy(np.array([fs[i] for i in order], np.uint8)).cuda()
    masks = torch.zeros(n, 112, dtype=torch.int64, device="cuda")
    values = torch.zeros(n, 112, dtype=torch.float32, device="cuda")
    times = []
    for r in range(args.reps + 1):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.check(lib.b200_op_encode_positions(d_boards.data_ptr(), d_offsets.data_ptr(), d_fs.data_ptr(), n, 2, 1,
                                                masks.data_ptr(), values.data_ptr(), None, None))
        e1.record()
        torch.cuda.synchronize()
        if r > 0 or args.reps == 0:
            times.append(e0.elapsed_time(e1))
    ms = float(np.median(times))
    nbytes = boards.nbytes + offsets.nbytes + n + n * 112 * 12
    print("encode_positions   n=%-7d boards=%-8d %8.3f ms  %8.1f GB/s (%d bytes read + written)  %.1f M positions/s"
          % (n, len(boards), ms, nbytes / ms / 1e6, nbytes, n / ms / 1e3), flush=True)
    return 0


def mux_bench(args):
    """Caller threads with small requests, through the aggregator and straight to the network."""
    import threading
    import time
    from . import mknet, network
    net = mknet.make_net(args.config)
    nw = network.Network(net, dict(max_batch=1024, precision=args.precision, slots=2))
    rng = np.random.default_rng(0)
    masks = rng.integers(0, 2 ** 62, size=(args.request, 112), dtype=np.int64).astype(np.uint64)
    values = np.ones((args.request, 112), np.float32)
    per_thread = 24

    def run(fn):
        def worker():
            for _ in range(per_thread):
                fn(masks, values)
        ths = [threading.Thread(target=worker) for _ in range(args.threads)]
        t0 = time.time()
        for t in ths:
            t.start()
        for t in ths:
            t.join()
        return args.threads * per_thread * args.request / (time.time() - t0)

    mux = nw.new_mux(max_batch=1024, wait_us=300)
    run(mux.evaluate)  # warm-up (graphs of the batch sizes that occur)
    before = mux.stats()
    merged = run(mux.evaluate)
    st = mux.stats()
    launches = st["batches"] - before["batches"]
    print("mux: %d threads x %d-position requests: %.0f evals/s, %.0f positions per launch"
          % (args.threads, args.request, merged, (st["positions"] - before["positions"]) / max(1, launches)), flush=True)
    mux.close()
    direct = run(nw.evaluate)
    print("direct: the same requests one computation each: %.0f evals/s" % direct, flush=True)
    nw.close()
    return 0


def multi_bench(args):
    """b200_multi_eval_host: --batch positions per GPU in one call, host buffers, replicated weights."""
    import time
    from . import mknet, network
    net = mknet.make_net(args.config)
    gpus = list(range(args.gpus))
    mg = network.MultiGpuNetwork(net, dict(max_batch=args.batch, precision=args.precision, slots=1), gpus=gpus)
    n = args.batch * len(gpus)
    rng = np.random.default_rng(0)
    masks = rng.integers(0, 2 ** 62, size=(n, 112), dtype=np.int64).astype(np.uint64)
    values = np.ones((n, 112), np.float32)
    for _ in range(3):
        mg.evaluate(masks, values)
    t0 = time.time()
    for _ in range(args.reps):
        mg.evaluate(masks, values)
    dt = (time.time() - t0) / args.reps
    print("multi: %d GPUs x %d positions per call: %.1f ms per call, %.0f evals/s (host buffers, one process)"
          % (len(gpus), args.batch, dt * 1e3, n / dt), flush=True)
    mg.close()
    return 0


def l2scratch_bench(lib, args):
    """b200_op_scratch_residency_probe: does a per-CTA scratch slice survive in L2 next to streaming traffic?"""
    from . import _lib
    ms = ctypes.c_float(0)
    _lib.check(lib.b200_op_scratch_residency_probe(args.slice_kb, args.stream_kb, args.iters, args.mode, ctypes.byref(ms)))
    sms = 148
    try:
        import torch
        sms = torch.cuda.get_device_properties(0).multi_processor_count
    except Exception:
        pass
    stream = sms * args.stream_kb * 1024.0 * args.iters
    scratch = 0.0 if args.mode & 8 else sms * args.slice_kb * 1024.0 * args.iters
    print("l2scratch slice_kb=%d stream_kb=%d iters=%d mode=%d: %.3f ms, footprint %.0f MB, moved %.0f GB/s through the "
          "SMs (stream %.1f GB + scratch written and read %.1f GB each)"
          % (args.slice_kb, args.stream_kb, args.iters, args.mode, ms.value, sms * args.slice_kb / 1024.0,
             (stream + 2 * scratch) / ms.value / 1e6, stream / 1e9, scratch / 1e9), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "encode", "mux", "multi", "l2scratch"])
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--slice-kb", type=int, default=1024)
    ap.add_argument("--stream-kb", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--mode", type=int, default=3)
    ap.add_argument("--threads", type=int, default=64)
    ap.add_argument("--request", type=int, default=16, help="positions per request (mux)")
    ap.add_argument("--config", default="cfg4")
    ap.add_argument("--batch", type=int, default=1024)
    ap.add_argument("--precision", default="fp16")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--only", default="")
    ap.add_argument("--fma", action="store_true", help="time the FMA kernel instead of the tensor-core kernel")
    ap.add_argument("--chain", type=int, default=1,
                    help="launches queued back to back between the two events (gemm): the time per launch then excludes "
                         "the host's launch latency, as in a graph replay")
    args = ap.parse_args()
    import torch
    from . import _lib
    lib = _lib.load()
    prec = _lib.PRECISIONS[args.precision]
    dt = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}[prec]
    if args.what == "encode":
        return encode_bench(lib, args)
    if args.what == "mux":
        return mux_bench(args)
    if args.what == "multi":
        return multi_bench(args)
    if args.what == "l2scratch":
        return l2scratch_bench(lib, args)
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
            if args.chain > 1:
                ms = ctypes.c_float(0)
                _lib.check(lib.b200_op_gemm_timed(A.data_ptr(), W.data_ptr(), b.data_ptr(), C.data_ptr(), M, N, K, 3,
                                                  prec, args.chain, ctypes.byref(ms), None))
                if r > 0 or args.reps == 0:
                    times.append(ms.value)
                continue
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
