"""Benchmark of the Qwen3-TTS decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one codec frame (16 code-predictor positions + one talker decode step) for
every session of the batch.  Workload: 64 concurrent sessions per GPU with ragged KV lengths
uniform in [64, 2048] over a paged bf16 KV cache (the batched configurations of the benchmark spec),
synthetic int8 per-channel weights of the real architecture, sampling T=0.9 / top-k 50 /
top-p 0.9.  Prints ONE JSON line:

  value      codec frames/s over all GPUs, frames enqueued back to back with all state resident
             in HBM (q3t_model_run_frames), timed with CUDA events, max over ranks
  e2e        the same metric through the drop-in C ABI the reference's host calls
             (qwen3_tts_model_batch_next_frame_begin_v2 + ..._finish_v2 per frame) with a host
             round trip per frame: frame table up, next tokens and codes down
  b1         the B=1 numbers (one session at KV length 512, the single-session configurations of the benchmark spec)
  roofline   the batch-1 int8 GEMV (configs[0], 2048 -> 6144) against the measured HBM peak
  cpu_baseline  the oracle's CPU restatement timed on this host's cores on a bounded sample

--impl reference times that CPU restatement as its own arm (the reference has no CPU
implementation of this path and its host is Rust, which this image cannot build).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SESSIONS = 64
GEMV_BYTES = 6144 * 2048 + 6144 * 4 + 2048 * 2 + 6144 * 2          # W + scales + x + y
TALKER_WEIGHT_BYTES = 1_423_966_208 + 2_322_432                      # int8 rows + fp32 scales
PREDICTOR_FRAME_BYTES = 1_323_302_912
KV_BYTES_PER_TOKEN = 28 * 2 * 1024 * 2                               # all layers, K and V


def frame_bytes(lengths) -> int:
    """Algorithmic HBM bytes of one lockstep frame: weights once, every session's KV once."""
    return TALKER_WEIGHT_BYTES + PREDICTOR_FRAME_BYTES + KV_BYTES_PER_TOKEN * int(sum(lengths))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, devices, enabled: bool = True):
        """One nvidia-smi process for all `devices` of the job (started by local rank 0 only: a
        process per rank, each initialising NVML on every GPU at the start of the timed region,
        perturbed an 8-rank run)."""
        self.devices = list(devices)
        self.enabled = enabled
        self.lines = []
        self.first = 0
        self.proc = None
        self.thread = None

    def start(self, ready_timeout_s: float = 5.0):
        """Starts sampling and returns once the first sample has arrived, so that the tool's
        start-up is over before the timed region begins."""
        if not self.enabled:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--id=" + ",".join(str(d) for d in self.devices),
                 f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()
        deadline = time.time() + ready_timeout_s
        while not self.lines and time.time() < deadline:
            time.sleep(0.01)

    def mark(self):
        """Samples from here on belong to the timed region."""
        self.first = len(self.lines)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.enabled:
            return None
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines[self.first:]:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "gpus_sampled": len(self.devices), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ CPU restatement, timed

def cpu_frame_seconds(repeats: int = 1):
    """Times the oracle (oracle/q3t_oracle.c, OpenMP over output rows) on a bounded sample of one
    B=1 frame -- one talker layer at KV length 513, one predictor layer, the heads and the
    sampler, with the real shapes -- and scales it to a whole frame (28 talker layers, 16 x 5
    predictor layers, 16 small projections and heads).  Returns (seconds per frame, threads,
    description)."""
    from oracle import oracle as o
    o.build()
    # all the host threads this process may use, whatever OMP_NUM_THREADS says (torchrun sets it
    # to 1 for its workers; only rank 0 runs the CPU arm)
    try:
        o.set_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        o.set_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(0)

    def layer(hidden, inter, qw, kvw):
        def q(n, k):
            return (rng.integers(-127, 128, size=(n, k), dtype=np.int8),
                    (rng.uniform(0.5, 1.5, size=n) / (73.6 * np.sqrt(k))).astype(np.float32))
        ones = o.to_bf16(np.ones(hidden, dtype=np.float32))
        hd = o.to_bf16(np.ones(128, dtype=np.float32))
        return dict(input_norm=ones, qkv=q(qw + 2 * kvw, hidden), o=q(hidden, qw), q_norm=hd,
                    k_norm=hd, post_norm=ones, gate_up=q(2 * inter, hidden), down=q(hidden, inter))

    talker = layer(2048, 6144, 2048, 1024)
    predictor = layer(1024, 3072, 2048, 1024)
    kc = o.to_bf16(rng.standard_normal((513, 1024)).astype(np.float32))
    vc = o.to_bf16(rng.standard_normal((513, 1024)).astype(np.float32))
    pk = np.zeros((16, 1024), dtype=np.uint16)
    pv = np.zeros((16, 1024), dtype=np.uint16)
    h = o.to_bf16(rng.standard_normal(2048).astype(np.float32))
    ph = o.to_bf16(rng.standard_normal(1024).astype(np.float32))
    head_w = rng.integers(-127, 128, size=(3072, 2048), dtype=np.int8)
    head_s = np.full(3072, 1.0 / 3000.0, dtype=np.float32)
    phead_w = rng.integers(-127, 128, size=(2048, 1024), dtype=np.int8)
    mtp_w = rng.integers(-127, 128, size=(1024, 2048), dtype=np.int8)
    pdims = o.predictor_dims(128)

    def timed(fn):
        best = None
        for _ in range(max(1, repeats)):
            t0 = time.perf_counter()
            fn()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        return best

    t_talker = timed(lambda: o.decoder_layer(h, talker, o.TALKER_DIMS, kc, vc, 512))
    t_pred = timed(lambda: o.decoder_layer(ph, predictor, pdims, pk, pv, 8))
    t_head = timed(lambda: o.sample(o.int8_gemm_rows(head_w, head_s, h)[0], 1, suppress=True,
                                    top_k=50, top_p=0.9))
    t_phead = timed(lambda: o.sample(o.int8_gemm_rows(phead_w, head_s[:2048], ph)[0], 1, top_k=50))
    t_mtp = timed(lambda: o.int8_gemm_rows(mtp_w, head_s[:1024], h))
    t_text = 2 * timed(lambda: o.int8_gemm_rows(head_w[:2048], head_s[:2048], h))
    frame = 28 * t_talker + 16 * 5 * t_pred + t_head + 15 * t_phead + 16 * t_mtp + t_text
    sample = ("1 talker layer (L=513) + 1 predictor layer + heads + samplers of a B=1 frame, real "
              "shapes, scaled x28 / x80 / x16 to one frame")
    return frame, o.threads(), sample


def run_reference_arm(args, rank: int) -> None:
    """CPU arm: the restatement of the reference's kernels on this host's cores."""
    if rank != 0:
        return
    for _ in range(max(0, min(args.warmup, 2))):
        cpu_frame_seconds()
    times = [cpu_frame_seconds()[0] for _ in range(max(1, min(args.steps, 5)))]
    frame_s = float(np.mean(times))
    _, threads, sample = cpu_frame_seconds()
    value = 1.0 / frame_s
    line = {
        "impl": "reference", "metric": "codec frames/s", "value": value, "unit": "frames/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": frame_s * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 weights x bf16 activations, fp32 accumulate",
        "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "frames/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation of this path and no Rust toolchain is "
                "available; this is the C restatement of its kernels (oracle/), frames are "
                "sequential on the CPU so the rate does not grow with the session count",
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int):
    return {"workload": "64 lockstep sessions/GPU, talker (28 layers, 2048 hidden) + code predictor "
                        "(5 layers, 16 positions) per frame, ragged KV U[64,2048], 16-token paged "
                        "bf16 KV, int8 per-channel weights, T=0.9 top-k 50 top-p 0.9",
            "sessions_per_gpu": SESSIONS, "global_sessions": SESSIONS * n_gpus,
            "kv_lengths": "randint(64, 2048, seed 3), the same draw on every GPU; session seeds differ per rank", "parallelism": f"dp{n_gpus}",
            "l2": "inputs larger than L2: 2.7 GB of weights and ~7.7 GB of KV per frame stream "
                  "from HBM; the predictor's 112 MB weight set may stay L2-resident across its 16 "
                  "positions, which is inherent to the workload"}


def percentile(values, q):
    return float(np.percentile(np.asarray(values, dtype=np.float64), q)) if len(values) else None


def make_sessions(q3t, model, count, lengths, frames_needed, talker_cfg, predictor_cfg, seed0):
    sessions = []
    for i in range(count):
        cap = min(8192, (int(lengths[i]) + frames_needed + 16 + 15) // 16 * 16)
        s = model.create_session(cap, seed0 + i)
        s.talker_sampling = talker_cfg
        s.predictor_sampling = predictor_cfg
        s.synthetic_prefill(int(lengths[i]), seed0 + i)
        sessions.append(s)
    return sessions


def api_frames(model, sessions, frames, trailing=11):
    """The call sequence of the reference's host: one lockstep begin, then every session's finish."""
    for _ in range(frames):
        if len(sessions) == 1:
            sessions[0].next_frame(trailing)
        else:
            pending = model.batch_begin_device_frames(sessions, [trailing] * len(sessions))
            for p in pending:
                p.finish_without_consumer()


def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); "
                         "use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    q3t = importlib.import_module("qwen3-tts-native_b200")
    synth = importlib.import_module("qwen3-tts-native_b200.synth")
    dp = importlib.import_module("qwen3-tts-native_b200.dp")
    native = q3t.native

    if args.leg == "gemv":
        # operator microbenchmark: no model needed (keeps ncu captures small)
        if args.gemv_mode is not None:
            native.set_gemv_mode(args.gemv_mode)
        g = native.benchmark_int8_gemv(local_rank, args.gemv_in, args.gemv_out, rows=args.rows,
                                       buffers=16, iterations=max(args.steps, 1))
        print(json.dumps({"leg": "gemv", "in": args.gemv_in, "out": args.gemv_out, "rows": args.rows,
                          "gemv_mode": native.set_gemv_mode(-1),
                          "us_per_launch": g.mean_launch_microseconds,
                          "cold_us": g.cold_launch_microseconds,
                          "GBps": (args.gemv_in * args.gemv_out) / g.mean_launch_microseconds / 1e3}),
              flush=True)
        return
    model = q3t.NativeTalkerModel.load(local_rank, synth.checkpoint_cuda(local_rank, seed=0))
    model.set_option("mask_eos", 1)
    model.set_option("batch_host_codes", 1)
    talker_cfg = q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.0)
    predictor_cfg = q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.0)
    K, W = args.steps, args.warmup
    total_frames = 3 * (K + W) + 8

    if args.leg != "all":
        # single legs, for profiling runs (ncu wants few launches and a small footprint)
        out = {"leg": args.leg}
        if True:
            count = 1 if args.leg == "b1" else SESSIONS
            lens = [512] if args.leg == "b1" else list(
                np.random.default_rng(3).integers(64, 2049, size=SESSIONS))
            ss = make_sessions(q3t, model, count, lens, K + W + 8, talker_cfg, predictor_cfg, 77)
            model.run_frames(ss, W, trailing_text_id=11)
            ms, _ = model.run_frames(ss, K, trailing_text_id=11)
            out.update(ms_per_frame=ms / K, frames_per_s=count * K / (ms * 1e-3))
            for s in ss:
                s.close()
        print(json.dumps(out), flush=True)
        model.close()
        return

    lengths = dp.shard_kv_lengths(rank, SESSIONS, per_rank=False)   # configs[3]: replicated per GPU
    sessions = make_sessions(q3t, model, SESSIONS, lengths, total_frames, talker_cfg, predictor_cfg,
                             dp.shard_session_seeds(rank, SESSIONS)[0])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident frame loop -----------------------------------------------------
    model.run_frames(sessions, W, trailing_text_id=11)
    launches_before = model.kernel_launches()
    clocks = ClockSampler(range(world), enabled=(rank == 0))
    clocks.start()
    barrier()
    clocks.mark()
    total_ms, per_frame = model.run_frames(sessions, K, trailing_text_id=11, want_frame_ms=True)
    barrier()
    clock_report = clocks.stop()
    launches = model.kernel_launches() - launches_before
    value, elapsed_s, _ = dp.whole_job_throughput(total_ms * 1e-3, SESSIONS * K, world, device="cuda")

    # ---- the same loop through the public C ABI, host round trip per frame ------------------
    # The caller is the library's compiled host pump (the reference's host is compiled Rust); the
    # same sequence driven from Python is reported beside it.
    model.host_pump_frames(sessions, W, trailing_text_id=11)
    barrier()
    pump_ms = model.host_pump_frames(sessions, K, trailing_text_id=11)
    torch.cuda.synchronize()
    e2e_value, _, _ = dp.whole_job_throughput(pump_ms * 1e-3, SESSIONS * K, world, device="cuda")
    barrier()
    t0 = time.perf_counter()
    api_frames(model, sessions, K)
    torch.cuda.synchronize()
    py_value, _, _ = dp.whole_job_throughput(time.perf_counter() - t0, SESSIONS * K, world, device="cuda")
    table_bytes = 64 * (3 * 4 + 8 * 8 + 2 * 20)      # sizeof(FrameTable)
    e2e = {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": table_bytes,
           "d2h_bytes_per_step": SESSIONS * (4 + 32),
           "api": "qwen3_tts_model_batch_next_frame_begin_v2 + qwen3_tts_session_next_frame_finish_v2",
           "caller": "q3t_host_pump_frames (C++ loop over the exported ABI)",
           "value_from_python_ctypes": py_value}

    lengths_now = [int(l) + W for l in lengths]
    fbytes = frame_bytes(lengths_now)
    hbm_peak, peak_kind = measured_peaks()
    frame_s = elapsed_s / K
    line = {
        "metric": "codec frames/s", "value": value, "unit": "frames/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": frame_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 weights x bf16 activations, fp32 accumulate", "data": "synthetic",
        "config": workload_config(world), "clocks": clock_report, "e2e": e2e,
        "gpu_launches": int(launches),
        "frame_latency_ms": {"p50": percentile(per_frame, 50), "p99": percentile(per_frame, 99)},
        "frame_roofline": {"bound": "hbm", "achieved": fbytes / frame_s / 1e9, "peak": hbm_peak,
                           "unit": "GB/s", "frac": fbytes / frame_s / 1e9 / hbm_peak,
                           "algorithmic_bytes_per_frame": fbytes, "peak_kind": peak_kind,
                           "frac_of_8TBs": fbytes / frame_s / 8.0e12},
    }
    for s in sessions:
        s.close()

    if rank == 0:
        # ---- B=1: one session at KV length 512 (configs[1] + configs[2]) ------------------------
        one = make_sessions(q3t, model, 1, [512], 2 * (K + W) + 80, talker_cfg, predictor_cfg, 77)
        k1 = max(K, 50)
        model.run_frames(one, W, trailing_text_id=11)
        torch.cuda.synchronize()
        ms1, per1 = model.run_frames(one, k1, trailing_text_id=11, want_frame_ms=True)
        model.host_pump_frames(one, W, trailing_text_id=11)
        torch.cuda.synchronize()
        api1 = model.host_pump_frames(one, K, trailing_text_id=11) * 1e-3
        torch.cuda.synchronize()
        b1_bytes = frame_bytes([513 + W])
        line["b1"] = {"value": k1 / (ms1 * 1e-3), "unit": "frames/s", "ms_per_frame": ms1 / k1,
                      "e2e_value": K / api1, "p50_ms": percentile(per1, 50), "p99_ms": percentile(per1, 99),
                      "roofline_frac": b1_bytes / (ms1 * 1e-3 / k1) / 1e9 / hbm_peak,
                      "frac_of_8TBs": b1_bytes / (ms1 * 1e-3 / k1) / 8.0e12,
                      "api": "qwen3_tts_session_next_frame"}
        one[0].close()
        # ---- a 128-position prompt (time to the first semantic token), 64 positions per pass ----
        ids = [int(t) for t in np.random.default_rng(4).integers(0, 151936, size=128)]
        prompt_ms = []
        for _ in range(3):
            ps = model.create_session(2048, 5)
            ps.talker_sampling, ps.predictor_sampling = talker_cfg, predictor_cfg
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ps.prefill(ids, [-1] * 128)
            prompt_ms.append((time.perf_counter() - t0) * 1e3)
            ps.close()
        line["prefill"] = {"positions": 128, "ms": min(prompt_ms), "positions_per_pass": 64,
                           "api": "qwen3_tts_session_prefill"}
        # ---- configs[4]: a 128-id prompt, then 375 frames (30 s of audio at 12.5 frames/s), B=1 and B=64;
        # the end-of-sequence code stays masked so that all 375 frames run on synthetic weights
        stream = {}
        for count in (1, SESSIONS):
            group = []
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for i in range(count):
                ps = model.create_session(640, 9000 + i)
                ps.talker_sampling, ps.predictor_sampling = talker_cfg, predictor_cfg
                ps.prefill(ids, [-1] * 128)
                group.append(ps)
            torch.cuda.synchronize()
            prompts_ms = (time.perf_counter() - t0) * 1e3
            total_ms, per = model.run_frames(group, 375, trailing_text_id=11, want_frame_ms=True)
            stream[f"b{count}"] = {"frames": 375, "prompt_ms_all_sessions": prompts_ms,
                                   "first_frame_ms": float(per[0]) if len(per) else None,
                                   "p50_ms": percentile(per, 50), "p99_ms": percentile(per, 99),
                                   "frames_per_s": count * 375 / (total_ms * 1e-3)}
            for ps in group:
                ps.close()
        line["stream_375_frames"] = stream
        # ---- batch-1 int8 GEMV, configs[0]: 16 weight images (201 MB > L2) round-robin --------------
        g = native.benchmark_int8_gemv(local_rank, 2048, 6144, rows=1, buffers=16, iterations=4000)
        gemv_s = g.mean_launch_microseconds * 1e-6
        line["roofline"] = {"bound": "hbm", "kernel": "gemv_b1_kernel<4> 2048->6144 (configs[0])",
                            "achieved": GEMV_BYTES / gemv_s / 1e9, "peak": hbm_peak, "unit": "GB/s",
                            "frac": GEMV_BYTES / gemv_s / 1e9 / hbm_peak, "peak_kind": peak_kind,
                            "frac_of_8TBs": GEMV_BYTES / gemv_s / 8.0e12,
                            "us_per_launch": g.mean_launch_microseconds, "traffic": 12639488,  # dram__bytes_read+write per launch, ncu capture of this kernel (profiles/)
                            "bytes_per_launch": GEMV_BYTES}
        if world == 1 and not args.no_cpu_baseline:
            frame_cpu, threads, sample = cpu_frame_seconds()
            line["cpu_baseline"] = {"value": 1.0 / frame_cpu, "unit": "frames/s", "cores": threads,
                                    "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    model.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemv-mode", type=int, default=None,
                    help="kernel for 1..8 rows: 0 SIMT, 1 mma.sync (default), 2 bulk-copy SIMT")
    ap.add_argument("--leg", choices=["all", "b64", "b1", "gemv"], default="all",
                    help="profiling aid: run one leg only and print a short JSON line")
    ap.add_argument("--gemv-in", type=int, default=2048)
    ap.add_argument("--gemv-out", type=int, default=6144)
    ap.add_argument("--rows", type=int, default=1)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
