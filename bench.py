#!/usr/bin/env python
"""Benchmark of the lc0 NN-evaluation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--precision fp16|bf16|fp32]
    python bench.py --impl reference ...      # the reference's own CPU (blas) backend on the host cores

One step = one evaluation of a batch of `--batch` positions (default 1024) per GPU with the seeded
BT4-class network (15 encoder layers, embedding 1024, 32 heads, dff 1536, smolgen) -- the configuration
the headline metric is quoted on.  Data are synthetic: seeded random-init weights and seeded random
legal playouts (tests/golden/positions_fmt2_*.npz).  With N > 1 (launched by torch.distributed.run, one
rank per GPU) every rank evaluates its own batch with replicated weights; there is no collective on the
data path, only a barrier and a max-reduction of the measured time.

`value` is timed with CUDA events on the evaluation stream with inputs resident in device memory; `e2e`
is timed through the NetworkComputation-style API with host buffers (H2D + D2H inside the timed region).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL_DENSE_TFLOPS = 2250.0  # B200 dense fp16 / bf16 tensor throughput as specified (not measured)
METRIC = "nn_evals_per_sec"
UNIT = "evals/s"
NET = "cfg4"
# configuration -> (network, batch per step, position set, precision, description)
CONFIGS = {
    "cfg1": ("cfg1", 64, 1, "fp32", "residual CNN 10x128 + SE, classical policy, WDL"),
    "cfg2": ("cfg2", 256, 1, "fp16", "residual CNN 20x256 + SE, convolutional policy (80 planes), WDL + moves-left"),
    "cfg3": ("cfg3", 512, 2, "fp16", "attention body 10 layers, embedding 256, 8 heads, dff 512, Mish, attention policy"),
    "cfg4": ("cfg4", 1024, 2, "fp16", "BT4-class net: 15 encoder layers, embedding 1024, 32 heads, dff 1536, smolgen "
                                      "32/256/256, attention policy, WDL + moves-left"),
    "cfg5": ("cfg4", 8192, 2, "fp16", "BT4-class net (as cfg4), 8192 positions per step split evenly over the GPUs, "
                                      "50/50 opening / late-middlegame positions"),
}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(tflops_sustained=p["bf16_tflops_sustained"], tflops_burst=p["bf16_tflops"],
                    hbm_gbs=p["hbm_gbs"], source="measured")
    return dict(tflops_sustained=1400.0, tflops_burst=1590.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc = None
        self.lines = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [l for (t, l) in self.lines if t0 <= t <= t1 + 0.2] or [l for (_, l) in self.lines]
        for line in rows:
            f = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(f[0]))
                mx = max(mx, float(f[1]))
            except Exception:
                continue
            for nme, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nme)
        if not sm:
            return None
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def load_positions(rank, batch, fmt=2, split=False, with_moves=False):
    if fmt == 1:
        name = "positions_fmt1_uniform.npz"
    else:
        name = "positions_fmt2_split.npz" if (split or rank % 2 == 1) else "positions_fmt2_uniform.npz"
    p = np.load(os.path.join(ROOT, "tests", "golden", name))
    masks, values = p["masks"], p["values"]
    reps = -(-batch // masks.shape[0])
    masks = np.tile(masks, (reps, 1))[:batch]
    values = np.tile(values, (reps, 1))[:batch]
    roll = lambda a: np.ascontiguousarray(np.roll(a, rank * 17, axis=0))
    if with_moves:
        legal = np.tile(p["legal"], (reps, 1))[:batch]
        legal = np.where(legal < 0, 0, legal).astype(np.uint16)
        n_legal = np.tile(p["n_legal"], reps)[:batch].astype(np.int32)
        return roll(masks), roll(values), roll(legal), roll(n_legal)
    return roll(masks), roll(values)


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's own blas backend (oracle/_ref/ref_eval, built from the reference
# sources by oracle/build_ref.py) or, when that binary is absent, the numpy port in oracle/.
# ------------------------------------------------------------------------------------------------
def cpu_reference(sample_positions, repeats, threads=None):
    from lc0_b200 import mknet, netproto, weights
    threads = threads or os.cpu_count() or 1
    masks, values = load_positions(0, sample_positions)
    ref_bin = os.path.join(ROOT, "oracle", "_ref", "ref_eval")
    net = mknet.make_net(NET)
    if os.path.exists(ref_bin):
        with tempfile.TemporaryDirectory() as tmp:
            npath = os.path.join(tmp, "net.pb")
            netproto.write_net(npath, net, compress=False)
            ppath = os.path.join(tmp, "p.pos")
            with open(ppath, "wb") as f:
                f.write(b"LC0POS1\0")
                f.write(np.array([sample_positions, 2], "<i4").tobytes())
                f.write(masks.astype("<u8").tobytes())
                f.write(values.astype("<f4").tobytes())
                f.write(np.zeros(sample_positions, "<i4").tobytes())
                f.write(np.zeros(sample_positions, "<i4").tobytes())
                f.write(np.full((sample_positions, 256), -1, "<i2").tobytes())
            r = subprocess.run([ref_bin, "blas", npath, ppath, "-", "threads=%d,batch_size=%d" % (threads, sample_positions),
                                str(repeats)], capture_output=True, text=True)
            if r.returncode == 0 and "evals_per_s=" in r.stdout:
                v = float(r.stdout.split("evals_per_s=")[1].split()[0])
                return dict(value=v, unit=UNIT, cores=threads, kind="reference",
                            sample="%d positions x %d repeats of the %s net through the reference blas backend "
                                   "(OpenBLAS, %d threads)" % (sample_positions, repeats, NET, threads))
    from oracle import oracle
    meta, t = weights.flatten(netproto.parse_net(netproto.encode("Net", net)))
    oracle.forward(meta, t, masks[:2], values[:2])
    t0 = time.time()
    for _ in range(repeats):
        oracle.forward(meta, t, masks, values)
    dt = time.time() - t0
    return dict(value=sample_positions * repeats / dt, unit=UNIT, cores=threads, kind="port",
                sample="%d positions x %d repeats of the %s net through the numpy port of the blas backend"
                       % (sample_positions, repeats, NET))


def reference_cuda_eval(net_name, runs, pos_fmt, backend, opts=""):
    """The reference's own CUDA backend (oracle/_ref/ref_eval_cuda: cuBLAS GEMMs + lc0's SIMT kernels, built for sm_100
    from the reference sources by `oracle/build_ref.py --cuda`) on this GPU through lc0's NetworkComputation API with
    host buffers.  `runs` is a list of (batch, repeats); returns one dict(value, p50_ms, p99_ms) or
    dict(unavailable=why) per run."""
    from lc0_b200 import mknet, netproto
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_eval_cuda")
    if not os.path.exists(exe):
        return [{"unavailable": "oracle/_ref/ref_eval_cuda is not built"} for _ in runs]
    out = []
    with tempfile.TemporaryDirectory() as tmp:
        npath, ppath = os.path.join(tmp, "net.pb"), os.path.join(tmp, "p.pos")
        netproto.write_net(npath, mknet.make_net(net_name), compress=False)
        for batch, repeats in runs:
            masks, values = load_positions(0, batch, pos_fmt)
            with open(ppath, "wb") as f:
                f.write(b"LC0POS1\0")
                f.write(np.array([batch, pos_fmt], "<i4").tobytes())
                f.write(masks.astype("<u8").tobytes())
                f.write(values.astype("<f4").tobytes())
                f.write(np.zeros(2 * batch, "<i4").tobytes())
                f.write(np.full((batch, 256), -1, "<i2").tobytes())
            try:
                r = subprocess.run([exe, backend, npath, ppath, "-",
                                    # the reference captures CUDA graphs for every batch size up to its mini-batch
                                    # size (2 x SM count = 296, network_cuda.cc:633-648,1041-1044) and fails with
                                    # "invalid argument" when max_batch is smaller than that
                                    "max_batch=%d%s" % (max(batch, 512), "," + opts if opts else ""),
                                    str(max(1, repeats))],
                                   capture_output=True, text=True, timeout=600)
            except subprocess.TimeoutExpired:
                out.append({"unavailable": "ref_eval_cuda did not finish within 600 s"})
                continue
            if r.returncode != 0 or "evals_per_s=" not in r.stdout:
                out.append({"unavailable": (r.stderr or r.stdout).strip()[-300:]})
                continue
            field = lambda k: float(r.stdout.split(k + "=")[1].split()[0]) if k + "=" in r.stdout else None
            out.append({"value": field("evals_per_s"), "p50_ms": field("p50_ms"), "p99_ms": field("p99_ms"),
                        "batch": batch, "backend": backend, "repeats": repeats})
    return out


def run_reference_cuda(args, rank):
    """--impl reference-cuda (extra, not part of the driver contract): the reference's own CUDA backend on the same
    GPU, same network, same batch."""
    if rank != 0:
        return
    net_name, cfg_batch, pos_fmt, cfg_prec, cfg_desc = CONFIGS[args.config]
    B = args.batch or cfg_batch
    backend = "cuda" if (args.precision or cfg_prec) == "fp32" else "cuda-fp16"
    res = reference_cuda_eval(net_name, [(B, args.steps)], pos_fmt, backend, args.ref_opts)[0]
    if "unavailable" in res:
        print(json.dumps({"impl": "reference-cuda", "unavailable": res["unavailable"]}))
        return
    v = res["value"]
    print(json.dumps({"impl": "reference-cuda", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": 1,
                      "steps": args.steps, "ms_per_step": 1000.0 * B / v, "dtype": "fp16" if backend == "cuda-fp16" else "fp32",
                      "config": {"workload": "%s: %s; batch %d; reference backend %s" % (args.config, cfg_desc, B, backend)},
                      "latency": {"batch": B, "p50_ms": res["p50_ms"], "p99_ms": res["p99_ms"]},
                      "e2e": {"value": v, "unit": UNIT}}), flush=True)


def run_reference(args, rank):
    """--impl reference: the reference's CPU implementation on the host cores.  One step = one evaluation of
    a 32-position sample (ref_eval performs one untimed warm-up evaluation itself before the timed repeats);
    ranks other than 0 exit without work."""
    if rank != 0:
        return
    sample = 32
    t0 = time.time()
    base = cpu_reference(sample, max(1, args.steps))
    dt = time.time() - t0
    v = base["value"]
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * sample / v, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "BT4-class net: 15 encoder layers, embedding 1024, 32 heads, dff 1536, smolgen "
                                   "32/256/256; reference CPU backend, %d-position sample per step" % sample,
                       "wall_seconds_including_load": dt},
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="cfg4", choices=sorted(CONFIGS))
    ap.add_argument("--batch", type=int, default=0, help="positions per GPU per step (default: the configuration's)")
    ap.add_argument("--precision", default="", help="fp16 | bf16 | fp32 (default: the configuration's)")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-cuda", action="store_true",
                    help="skip the reference's CUDA backend on the same GPU (reported as `reference_cuda`)")
    ap.add_argument("--ref-opts", default="", help="extra backend options for --impl reference-cuda")
    ap.add_argument("--net-options", default="", help="extra options for the network, e.g. fused_se=0,fold_ln=0")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return 0
    if args.impl == "reference-cuda":
        run_reference_cuda(args, rank)
        return 0

    import torch
    import torch.distributed as dist
    from lc0_b200 import mknet, network, sharding

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    net_name, cfg_batch, pos_fmt, cfg_prec, cfg_desc = CONFIGS[args.config]
    if not args.precision:
        args.precision = cfg_prec
    if not args.batch:
        args.batch = cfg_batch // world if args.config == "cfg5" else cfg_batch
    # The reference's own GPU backend on this GPU, before anything of ours is resident: the same network at the
    # benchmark's batch and at batch 256 (throughput and per-evaluation latency through lc0's API, host buffers).
    ref_cuda = None
    if world == 1 and rank == 0 and not args.no_reference_cuda and args.precision != "fp32":
        ref_cuda = {"what": "the reference's cuda-fp16 backend (cuBLAS + lc0's own kernels, compiled for sm_100 from "
                            "the reference sources) on the same GPU, NetworkComputation API with host buffers"}
        sizes = sorted({args.batch, min(256, args.batch)}, reverse=True)
        for b_ref, res in zip(sizes, reference_cuda_eval(net_name, [(b, 10 if b >= 1024 else 40) for b in sizes],
                                                         pos_fmt, "cuda-fp16")):
            ref_cuda["batch_%d" % b_ref] = res
    net = mknet.make_net(net_name)
    # two workspace slots, as the lc0 plug-in creates the network: a second computation can stage its inputs and have
    # its graph queued while the first one's kernels run (the phases with two computations in flight need it)
    nw = network.Network(net, dict(network.parse_options(args.net_options), gpu=local_rank, max_batch=args.batch,
                                   precision=args.precision, slots=2))
    del net
    info = nw.info
    B = args.batch
    masks, values = load_positions(rank, B, pos_fmt, split=args.config == "cfg5")
    d_masks = torch.from_numpy(masks.view(np.int64)).cuda()
    d_values = torch.from_numpy(values).cuda()
    d_policy = torch.empty(B, 1858, dtype=torch.float32, device="cuda")
    d_qdm = torch.empty(B, 3, dtype=torch.float32, device="cuda")
    stream = torch.cuda.ExternalStream(nw.stream())

    def step_device():
        nw.enqueue_device(d_masks.data_ptr(), d_values.data_ptr(), B, d_policy.data_ptr(), d_qdm.data_ptr())

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing (value) ----
    for _ in range(args.warmup):
        step_device()
    nw.sync()
    status = nw.device_status()
    if status:
        raise RuntimeError("device status word = %d (a bounded wait gave up)" % status)
    barrier()
    sampler = ClockSampler(local_rank)
    time.sleep(0.25)
    l0 = nw.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record(stream)
    for _ in range(args.steps):
        step_device()
    e1.record(stream)
    nw.sync()
    t1 = time.time()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = nw.launch_count() - l0
    clocks = sampler.stop(t0, t1)
    # Per-kernel-class pass: the same K steps again with CUDA-event pairs around every launch (this pass launches
    # kernel by kernel; the timed pass above replays the captured graph of the same launches).  In this pass smolgen's
    # small dense layers run in line rather than on the side stream, so that every span times one kernel alone.
    nw.set_profiling(True)
    nw.get_profile(reset=True)
    nw.get_profile_tagged(reset=True)
    ep0, ep1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ep0.record(stream)
    for _ in range(args.steps):
        step_device()
    ep1.record(stream)
    nw.sync()
    prof = nw.get_profile(reset=True)
    tagged = nw.get_profile_tagged(reset=True)
    prof_ms = ep0.elapsed_time(ep1)
    nw.set_profiling(False)
    ms = sharding.gather_max(ms, dist if world > 1 else None)
    value = world * B * args.steps / (ms / 1000.0)

    # ---- end-to-end timing through the computation API (host buffers) ----
    def step_host():
        c = nw.new_computation()
        c.add_inputs(masks, values)
        c.compute_blocking()
        q = c.get_q_val(0)
        c.close()
        return q

    for _ in range(2):
        step_host()
    barrier()
    th0 = time.time()
    for _ in range(args.steps):
        step_host()
    torch.cuda.synchronize()
    th = time.time() - th0
    th = sharding.gather_max(th, dist if world > 1 else None)
    e2e_value = world * B * args.steps / th

    # The same K steps with two computations in flight, the way lc0 drives a backend (GetThreads() == 2: one
    # search thread fills and reads a batch while the other's batch is on the GPU); every step still does its own
    # host->device and device->host copies inside the timed region.
    def run_pipelined(step_fn, steps):
        import threading
        errs = []

        def worker(k):
            try:
                for _ in range(k):
                    step_fn()
            except Exception as e:  # noqa: BLE001 - reported to the main thread
                errs.append(e)

        ths = [threading.Thread(target=worker, args=(steps // 2 + (steps % 2 if i == 0 else 0),)) for i in range(2)]
        t0 = time.time()
        for t in ths:
            t.start()
        for t in ths:
            t.join()
        torch.cuda.synchronize()
        dt = time.time() - t0
        if errs:
            raise errs[0]
        return dt

    run_pipelined(step_host, 2)
    barrier()
    th2 = sharding.gather_max(run_pipelined(step_host, args.steps), dist if world > 1 else None)
    e2e_two = world * B * args.steps / th2

    # ---- the same with the legal-move softmax on the device and compact return (no 1858-logit vectors cross PCIe) ----
    _, _, legal, n_legal = load_positions(rank, B, pos_fmt, split=args.config == "cfg5", with_moves=True)

    def step_compact():
        c = nw.new_computation()
        c.set_policy_options(1.0, compact=True)
        c.add_inputs_with_moves(masks, values, legal, n_legal)
        c.compute_blocking()
        q = c.get_q_val(0)
        c.close()
        return q

    for _ in range(3):
        step_compact()
    barrier()
    tcs = sharding.gather_max(run_pipelined(step_compact, args.steps), dist if world > 1 else None)
    compact_value = world * B * args.steps / tcs

    # ---- the same with game histories as input: position encoding (EncodePositionForNN) and legal-move softmax on the
    # device; 88 bytes per history entry go up instead of 1344 bytes of planes per position ----
    enc_value = None
    enc_h2d = 0
    enc_path = os.path.join(ROOT, "tests", "golden", "encoder_golden.npz")
    if os.path.exists(enc_path) and info.input_format in (1, 2, 3, 4, 132):
        eg = np.load(enc_path)
        offs = eg["offsets"]
        # the last (at most 8) entries of each fixture history, tiled to the batch
        hists = []
        for s_ in range(len(eg["from_start"])):
            a, b = int(offs[s_]), int(offs[s_ + 1])
            first = max(a, b - 8)
            hists.append((np.ascontiguousarray(eg["boards"][first:b]), bool(eg["from_start"][s_]) and first == a))
        order = [(i + 17 * rank) % len(hists) for i in range(B)]
        h_boards = np.concatenate([hists[i][0] for i in order])
        h_offsets = np.concatenate([[0], np.cumsum([len(hists[i][0]) for i in order])]).astype(np.int32)
        h_from_start = np.array([hists[i][1] for i in order], np.uint8)
        enc_h2d = int(len(h_boards) * 88 + B * (256 * 2 + 4 + 4 + 1))

        def step_history():
            c = nw.new_computation()
            c.set_policy_options(1.0, compact=True)
            c.add_positions(h_boards, h_offsets, h_from_start, legal, n_legal)
            c.compute_blocking()
            q = c.get_q_val(0)
            c.close()
            return q

        for _ in range(2):
            step_history()
        barrier()
        tenc = sharding.gather_max(run_pipelined(step_history, max(2, args.steps // 2)),
                                   dist if world > 1 else None)
        enc_value = world * B * max(2, args.steps // 2) / tenc

    # ---- latency of one batch-256 computation through the same API (p50 / p99 over 40 calls) ----
    lat = None
    if B >= 256:
        m256, v256 = masks[:256], values[:256]

        def step256():
            c = nw.new_computation()
            c.add_inputs(m256, v256)
            c.compute_blocking()
            c.get_q_val(0)
            c.close()

        for _ in range(3):
            step256()
        samples = []
        for _ in range(40):
            t_a = time.perf_counter()
            step256()
            samples.append((time.perf_counter() - t_a) * 1000.0)
        lat = {"batch": 256, "p50_ms": float(np.percentile(samples, 50)), "p99_ms": float(np.percentile(samples, 99)),
               "calls": len(samples), "path": "NewComputation/AddInput/ComputeBlocking/GetQVal with host buffers"}

    if rank == 0:
        peaks = read_peaks()
        g = prof["gemm_tc"]
        achieved = g["work"] / (g["ms"] * 1e-3) / 1e12 if g["ms"] > 0 else 0.0
        total_ms = sum(v["ms"] for v in prof.values())
        roofline = {"bound": "tensor", "kernel": "gemm_tc_kernel (tcgen05 GEMM, all launches of the timed region)",
                    "achieved": achieved, "peak": peaks["tflops_sustained"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["tflops_sustained"], "peak_source": peaks["source"] + " sustained bf16",
                    "frac_of_burst_peak": achieved / peaks["tflops_burst"],
                    # the nominal dense fp16 / bf16 figure of the part, for context
                    "frac_nominal": achieved / NOMINAL_DENSE_TFLOPS, "nominal_peak": NOMINAL_DENSE_TFLOPS,
                    "launches": g["launches"], "share_of_step": g["ms"] / total_ms if total_ms else None,
                    # DRAM bytes of the largest launch of the class (QKV + smolgen compression, M = 64 * batch): read
                    # A once and W once, write C once.  An ncu capture of the same kernel at M = 8192 measured DRAM
                    # reads equal to A + W (profiles/gemm_tc_kernel_qkv_batch128.md); scaled by the rows processed.
                    "traffic": (float(B) * 64 * 1024 * 2 + 3104 * 1024 * 2 + float(B) * 64 * 3104 * 2)
                    if args.config in ("cfg4", "cfg5") else None,
                    "traffic_of": "the QKV launch (largest of the class), bytes per launch, scaled from an ncu capture",
                    "how": "CUDA-event pairs around every launch during a second pass of the same %d steps "
                           "(%.3f ms per step in that pass)" % (args.steps, prof_ms / args.steps)}
        other = {}
        for k in ("attention", "layer_norm"):
            v = prof[k]
            if v["ms"] > 0:
                gbs = v["work"] / (v["ms"] * 1e-3) / 1e9
                other[k] = {"GBps": gbs, "frac_hbm": gbs / peaks["hbm_gbs"], "ms_per_step": v["ms"] / args.steps,
                            "launches": v["launches"]}
        for k in ("gemm_tc", "gemm_fma", "other"):
            other.setdefault(k, {})["ms_per_step"] = prof[k]["ms"] / args.steps
            other[k]["launches"] = prof[k]["launches"]
        # the tensor-core products of the encoder layers one by one, timed in place (same pass)
        by_shape = {}
        for k in ("qkv", "out_proj", "ffn1", "ffn2", "smolgen_dense", "smolgen_bias", "embedding", "heads"):
            v = tagged.get(k)
            if v and v["launches"]:
                tf = v["work"] / (v["ms"] * 1e-3) / 1e12
                by_shape[k] = {"us_per_launch": 1000.0 * v["ms"] / v["launches"], "launches": v["launches"],
                               "TFLOPs": tf, "frac_sustained": tf / peaks["tflops_sustained"],
                               "frac_nominal": tf / NOMINAL_DENSE_TFLOPS, "ms_per_step": v["ms"] / args.steps}
        other["gemm_tc"]["by_shape"] = by_shape
        enc = [tagged[k] for k in ("qkv", "out_proj", "ffn1", "ffn2") if tagged.get(k) and tagged[k]["launches"]]
        if enc:
            tf = sum(v["work"] for v in enc) / (sum(v["ms"] for v in enc) * 1e-3) / 1e12
            other["gemm_tc"]["encoder_gemms"] = {"TFLOPs": tf, "frac_sustained": tf / peaks["tflops_sustained"],
                                                 "frac_burst": tf / peaks["tflops_burst"],
                                                 "frac_nominal": tf / NOMINAL_DENSE_TFLOPS,
                                                 "what": "QKV, output projection, FFN dense 1 and 2 of all layers"}
        if tagged.get("attention") and tagged["attention"]["launches"]:
            other.setdefault("attention", {})["us_per_launch"] = \
                1000.0 * tagged["attention"]["ms"] / tagged["attention"]["launches"]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": args.precision, "data": "synthetic",
            "config": {"workload": "%s: %s; batch %d per GPU" % (args.config, cfg_desc, B),
                       "batch_per_gpu": B, "global_batch": B * world, "parallelism": "replicated weights, batch split",
                       "l2": "per-step working set (weights %.2f GB + activations) exceeds the 126 MB L2"
                             % (info.weight_bytes / 1e9)},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(B * 112 * 12),
                    "d2h_bytes_per_step": int(B * (1858 + 3) * 4), "ms_per_step": 1000.0 * th / args.steps,
                    "how": "NewComputation/AddInput/ComputeBlocking/GetQVal with host buffers, one computation at a "
                           "time; wall clock over the K steps",
                    "two_computations_in_flight": e2e_two},
            "e2e_compact_policy": {"value": compact_value, "unit": UNIT,
                                   "h2d_bytes_per_step": int(B * (112 * 12 + 256 * 2 + 4)),
                                   "d2h_bytes_per_step": int(B * (256 * 4 + 12)),
                                   "what": "legal-move policy softmax on the device, only per-move probabilities "
                                           "returned; two computations in flight"},
            "e2e_history_input": None if enc_value is None else {
                "value": enc_value, "unit": UNIT, "h2d_bytes_per_step": enc_h2d,
                "d2h_bytes_per_step": int(B * (256 * 4 + 12)),
                "what": "positions given as game histories (last 8 boards), planes and legal-move softmax produced on "
                        "the device; two computations in flight"},
            "gpu_launches": int(launches),
            "roofline": roofline,
            "kernel_classes": other,
            "latency": lat,
            "reference_cuda": ref_cuda,
            "flops_per_eval": info.flops_per_position,
            "model_tflops": value / world * info.flops_per_position / 1e12,
        }
        if world == 1 and not args.no_cpu_baseline and args.config in ("cfg4", "cfg5"):
            line["cpu_baseline"] = cpu_reference(32, 4)
        print(json.dumps(line), flush=True)
    nw.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
