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
  cpu_baseline  the oracle's CPU restatement timed on this host's cores: whole B=1 frames, median
  existing_kernels  the reference project's own CUDA code on this GPU (oracle/_ref, test
             infrastructure, outside every timed region): its int8 GEMV kernel on configs[0] and its
             whole library's B=1 / B=8 frames through its ABI, with this library's times for the same
             calls beside them

--impl reference times the CPU restatement as its own arm (the reference has no CPU implementation
of this path and its host is Rust, which this image cannot build): whole B=1 frames, one per step.
--leg b64 | b1 | gemv | attn | existing run one part alone (profiling wants few launches and a
small footprint; `existing` drives whichever library QWEN3_TTS_TALKER_LIBRARY names).
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
GEMV_TRAFFIC_NCU = 12647936                                               # bytes per launch, see roofline.traffic_source
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
                 f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms",
                 # one GPU: a sample every 25 ms (the timed region is a fraction of a second); several
                 # GPUs: every 100 ms, since each sample queries every GPU of the job
                 "25" if len(self.devices) == 1 else "100"],
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

CPU_WORKLOAD = ("B=1 frames, one after the other, on the host cores: 28 talker layers at KV length 513, "
                "16 x 5 code-predictor layers, 16 input projections, 15 predictor heads + the codec head, "
                "2 text projections, 16 samplers (T=0.9 top-k 50 top-p 0.9), every operator executed at its "
                "real shape; a CPU runs sessions one at a time, so its frames/s is the single-session rate")


class CpuFrames:
    """The oracle (oracle/q3t_oracle.c, OpenMP over output rows) set up to run whole B=1 frames."""

    def __init__(self):
        from oracle import oracle as o
        o.build()
        # all the host threads this process may use, whatever OMP_NUM_THREADS says (torchrun sets it
        # to 1 for its workers; only rank 0 runs the CPU arm)
        try:
            o.set_threads(len(os.sched_getaffinity(0)))
        except (AttributeError, OSError):
            o.set_threads(os.cpu_count() or 1)
        self.o = o
        rng = np.random.default_rng(0)

        def layer(hidden, inter, qw, kvw):
            def q(n, k):
                return (rng.integers(-127, 128, size=(n, k), dtype=np.int8),
                        (rng.uniform(0.5, 1.5, size=n) / (73.6 * np.sqrt(k))).astype(np.float32))
            ones = o.to_bf16(np.ones(hidden, dtype=np.float32))
            hd = o.to_bf16(np.ones(128, dtype=np.float32))
            return dict(input_norm=ones, qkv=q(qw + 2 * kvw, hidden), o=q(hidden, qw), q_norm=hd,
                        k_norm=hd, post_norm=ones, gate_up=q(2 * inter, hidden), down=q(hidden, inter))

        self.talker = layer(2048, 6144, 2048, 1024)
        self.predictor = layer(1024, 3072, 2048, 1024)
        self.kc = o.to_bf16(rng.standard_normal((513, 1024)).astype(np.float32))
        self.vc = o.to_bf16(rng.standard_normal((513, 1024)).astype(np.float32))
        self.pk = np.zeros((16, 1024), dtype=np.uint16)
        self.pv = np.zeros((16, 1024), dtype=np.uint16)
        self.h = o.to_bf16(rng.standard_normal(2048).astype(np.float32))
        self.ph = o.to_bf16(rng.standard_normal(1024).astype(np.float32))
        self.head_w = rng.integers(-127, 128, size=(3072, 2048), dtype=np.int8)
        self.head_s = np.full(3072, 1.0 / 3000.0, dtype=np.float32)
        self.phead_w = rng.integers(-127, 128, size=(2048, 1024), dtype=np.int8)
        self.mtp_w = rng.integers(-127, 128, size=(1024, 2048), dtype=np.int8)
        self.pdims = o.predictor_dims(128)
        self.threads = o.threads()

    def frame(self) -> float:
        """Runs every operator of one B=1 frame (the same weights serve every layer: values do not
        change the time) and returns the seconds it took."""
        o = self
        lib = self.o
        t0 = time.perf_counter()
        for position in range(16):                       # code predictor: 16 positions x 5 layers
            lib.int8_gemm_rows(o.mtp_w, o.head_s[:1024], o.h)
            for _ in range(5):
                lib.decoder_layer(o.ph, o.predictor, o.pdims, o.pk, o.pv, position)
            if position > 0:
                lib.sample(lib.int8_gemm_rows(o.phead_w, o.head_s[:2048], o.ph)[0], 1, top_k=50, top_p=0.9)
        for _ in range(2):                               # trailing text: two 2048 x 2048 projections
            lib.int8_gemm_rows(o.head_w[:2048], o.head_s[:2048], o.h)
        for _ in range(28):                              # talker step at position 512
            lib.decoder_layer(o.h, o.talker, lib.TALKER_DIMS, o.kc, o.vc, 512)
        lib.sample(lib.int8_gemm_rows(o.head_w, o.head_s, o.h)[0], 1, suppress=True, top_k=50, top_p=0.9)
        return time.perf_counter() - t0


def cpu_frames_timed(frames: int, warmup: int, budget_s: float):
    """(per-frame seconds of the frames that ran, threads).  Stops early once `budget_s` is spent,
    but runs at least one timed frame."""
    cpu = CpuFrames()
    for _ in range(warmup):
        cpu.frame()
    times = []
    started = time.perf_counter()
    for _ in range(max(1, frames)):
        times.append(cpu.frame())
        if time.perf_counter() - started > budget_s:
            break
    return times, cpu.threads


def run_reference_arm(args, rank: int) -> None:
    """CPU arm: the restatement of the reference's kernels on this host's cores, whole frames."""
    if rank != 0:
        return
    times, threads = cpu_frames_timed(max(args.steps, 5), min(args.warmup, 2), budget_s=150.0)
    frame_s = float(np.median(times))
    value = 1.0 / frame_s
    config = workload_config(args.gpus)
    config["workload"] = CPU_WORKLOAD
    config["gpu_arm_workload"] = workload_config(args.gpus)["workload"]
    line = {
        "impl": "reference", "metric": "codec frames/s", "value": value, "unit": "frames/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": min(args.warmup, 2),
        "ms_per_step": frame_s * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 weights x bf16 activations, fp32 accumulate",
        "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": "frames/s", "cores": threads, "kind": "port",
                         "sample": f"{len(times)} whole B=1 frames, median; " + CPU_WORKLOAD},
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "frame_seconds": {"min": float(np.min(times)), "median": frame_s, "max": float(np.max(times))},
        "note": "the reference has no CPU implementation of this path and no Rust toolchain is "
                "available; this is the C restatement of its kernels (oracle/).  steps = whole frames "
                "actually run (the requested count, or fewer if 150 s were spent), value = 1 / median",
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


def abi_frame_times(q3t, model, talker_cfg, predictor_cfg, frames: int = 30):
    """B=1 and B=8 frame times through the reference's ABI calls only (session_create, prefill of a
    512-id prompt, session_next_frame / model_batch_next_frame_begin_v2 + finish_v2), wall clock with
    the host round trip every frame: works on any library that exports that ABI."""
    ids = [int(t) for t in np.random.default_rng(4).integers(0, 151936, size=512)]
    out = {"prompt_ids": 512, "frames_timed": frames}

    def start(count, seed0):
        group = []
        for i in range(count):
            s = model.create_session(1024, seed0 + i)
            s.talker_sampling, s.predictor_sampling = talker_cfg, predictor_cfg
            s.prefill(ids, [-1] * 512)
            group.append(s)
        return group

    one = start(1, 300)[0]
    gpu_ms, wall = [], []
    for f in range(frames + 3):
        if one.ended:
            break
        t0 = time.perf_counter()
        fr = one.next_frame(11)
        if f >= 3:
            wall.append((time.perf_counter() - t0) * 1e3)
            gpu_ms.append(fr.predictor_gpu_milliseconds + fr.talker_gpu_milliseconds)
    one.close()
    out["b1"] = {"api": "qwen3_tts_session_next_frame", "frames": len(wall),
                 "ms_per_frame_wall": percentile(wall, 50), "ms_per_frame_gpu_events": percentile(gpu_ms, 50)}
    group = start(8, 400)
    wall = []
    for f in range(frames + 3):
        if any(s.ended for s in group):
            break
        t0 = time.perf_counter()
        pending = model.batch_begin_device_frames(group, [11] * len(group))
        for p in pending:
            p.finish_without_consumer()
        if f >= 3:
            wall.append((time.perf_counter() - t0) * 1e3)
    for s in group:
        s.close()
    out["b8"] = {"api": "qwen3_tts_model_batch_next_frame_begin_v2 + qwen3_tts_session_next_frame_finish_v2",
                 "frames": len(wall), "ms_per_frame_wall": percentile(wall, 50),
                 "frames_per_s": 8e3 / percentile(wall, 50) if wall else None}
    return out


def existing_kernels_block():
    """The reference project's own CUDA code on this GPU, compiled for sm_100a into oracle/_ref (test
    infrastructure): its int8 GEMV kernel on configs[0], and its whole library (int8 decode switched
    on) driven through its ABI in a child process.  Outside every timed region of this line."""
    from oracle import oracle as o
    if not o.ref_available():
        return {"unavailable": "oracle/_ref not built (needs a checkout of the reference where it was built)"}
    o.build()
    block = {}
    us = o.ref_time_int8_gemm(2048, 6144, 1, 0, 16, 2000)
    block["int8_gemm_rows_2048x6144"] = {
        "kernel": "reference launch_int8_gemm_rows (int8_gemv.cu:318-334), rows = 1, 16 rotating weight images",
        "us_per_launch": us, "GBps": GEMV_BYTES / us / 1e3 if us > 0 else None}
    library = os.path.join(ROOT, "oracle", "_ref", "libqwen3_tts_cuda_ref.so")
    if not os.path.exists(library):
        block["library"] = {"unavailable": "oracle/_ref/libqwen3_tts_cuda_ref.so not built"}
        return block
    env = dict(os.environ)
    env.update({"QWEN3_TTS_TALKER_LIBRARY": library, "QWEN3_TTS_INT8_DECODE": "1"})
    for name in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(name, None)
    try:
        proc = subprocess.run([sys.executable, os.path.abspath(__file__), "--leg", "existing"], env=env,
                              capture_output=True, text=True, timeout=600)
        last = [l for l in proc.stdout.splitlines() if l.startswith("{")]
        if proc.returncode == 0 and last:
            block["library"] = json.loads(last[-1])
        else:
            block["library"] = {"unavailable": (proc.stderr or "no output")[-300:]}
    except (subprocess.TimeoutExpired, OSError) as e:
        block["library"] = {"unavailable": str(e)[:300]}
    return block


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
    if args.leg == "attn":
        # operator microbenchmark: the 64-session ragged batch of one talker layer, contiguous caches
        us, kv_bytes = native.benchmark_decode_attention(local_rank, rows=SESSIONS, min_length=64, max_length=2048,
                                                         seed=3, iterations=max(args.steps, 1))
        print(json.dumps({"leg": "attn", "rows": SESSIONS, "kv_lengths": "U[64, 2048], seed 3",
                          "us_per_launch": us, "kv_bytes": kv_bytes, "GBps": kv_bytes / us / 1e3}), flush=True)
        return
    gemv_runs = None
    if rank == 0 and args.leg == "all":
        # The operator microbenchmark of the roofline block, taken before the model is loaded (the
        # same state of the device as `--leg gemv`; with 12 GB of model and caches allocated first the
        # figure moved by up to 8 % from run to run): five runs of 2000 launches, sorted; the median
        # run is reported.
        gemv_runs = sorted((native.benchmark_int8_gemv(local_rank, 2048, 6144, rows=1, buffers=16, iterations=2000)
                            for _ in range(5)), key=lambda r: r.mean_launch_microseconds)
    model = q3t.NativeTalkerModel.load(local_rank, synth.checkpoint_cuda(local_rank, seed=0))
    talker_cfg = q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.0)
    predictor_cfg = q3t.SamplingConfig(True, 50, 0.9, 0.9, 1.0)
    if args.leg == "existing":
        # whichever library QWEN3_TTS_TALKER_LIBRARY names, through the reference's ABI only
        out = abi_frame_times(q3t, model, talker_cfg, predictor_cfg)
        out["library"] = os.path.basename(os.environ.get("QWEN3_TTS_TALKER_LIBRARY", "libqwen3_tts_cuda.so"))
        print(json.dumps(out), flush=True)
        model.close()
        return
    model.set_option("mask_eos", 1)
    model.set_option("batch_host_codes", 1)
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
        runs = gemv_runs
        g = runs[len(runs) // 2]
        gemv_s = g.mean_launch_microseconds * 1e-6
        line["roofline"] = {"bound": "hbm", "kernel": "gemv_mma_kernel<4,false,false,1> 2048->6144 (configs[0]); the kernel the B=1 frame "
                                      "dispatches for all its projections (gemv mode 1)",
                            "achieved": GEMV_BYTES / gemv_s / 1e9, "peak": hbm_peak, "unit": "GB/s",
                            "frac": GEMV_BYTES / gemv_s / 1e9 / hbm_peak, "peak_kind": peak_kind,
                            "frac_of_8TBs": GEMV_BYTES / gemv_s / 8.0e12,
                            "us_per_launch": g.mean_launch_microseconds,
                            # dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture
                            # summarised in profiles/gemv_mma_kernel_2048x6144_rows1.md (not measured by this run)
                            "traffic": GEMV_TRAFFIC_NCU, "traffic_source": "ncu capture, profiles/gemv_mma_kernel_2048x6144_rows1.md",
                            "bytes_per_launch": GEMV_BYTES,
                            "us_per_launch_runs": [r.mean_launch_microseconds for r in runs]}
        if world == 1 and not args.no_existing:
            line["existing_kernels"] = existing_kernels_block()
            line["existing_kernels"]["ours_same_calls"] = abi_frame_times(q3t, model, talker_cfg, predictor_cfg)
        if world == 1 and not args.no_cpu_baseline:
            cpu_times, threads = cpu_frames_timed(5, 1, budget_s=30.0)
            line["cpu_baseline"] = {"value": 1.0 / float(np.median(cpu_times)), "unit": "frames/s",
                                    "cores": threads, "kind": "port",
                                    "sample": f"{len(cpu_times)} whole B=1 frames, median; " + CPU_WORKLOAD}
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
    ap.add_argument("--no-existing", action="store_true",
                    help="skip the existing_kernels block (the reference's kernels and library from oracle/_ref)")
    ap.add_argument("--gemv-mode", type=int, default=None,
                    help="kernel for 1..8 rows: 0 SIMT, 1 int8 mma.sync (default)")
    ap.add_argument("--leg", choices=["all", "b64", "b1", "gemv", "attn", "existing"], default="all",
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
