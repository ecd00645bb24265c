"""Frame composition and prompt path against the reference project's own library, executed here.

oracle/_ref/libqwen3_tts_cuda_ref.so is the reference's whole talker library (its eight .cu files,
unmodified, compiled for sm_100a by oracle/build_ref.sh) under its own C ABI.  A worker process per
library (tests/reference_frames_worker.py) uploads the same 404 synthetic tensors, whose decode
matrices are exactly int8-representable, runs the same prompts and lockstep batches of 2 and 8
sessions through the same ABI calls, and reports first tokens, the 16 codes and the next semantic
token of every frame, the session counters, the parity-trace lines of the prompt and the layer-0
stage tensors.  The reference runs with QWEN3_TTS_INT8_DECODE=1: its lockstep batch path is then the
fused int8 path (talker.cu:2054-2333) whose semantics this library implements for every batch size.

What can and cannot be equal.  The reference's prompt path is bf16 cuBLAS with unfused residual
adds, a bf16-rounded SiLU and bf16-rounded attention probabilities (talker.cu:2750-3249); this
library runs the prompt through its int8 decode kernels.  On int8-exact weights both multiply the
same numbers, so stage tensors agree to bf16 rounding and drift apart by rounding flips only; the
KV cache each library decodes from is therefore its own prompt's, and exact code equality over many
frames is not implied.  The test asserts what the arithmetic guarantees (identical structure and
counters, stage tensors within a bf16 rounding step, hidden-state statistics and logits that
track) and records, in the file named by Q3T_PARITY_REPORT, how far the code sequences agree.

The frames themselves are pinned exactly another way: oracle/_ref/libqwen3_tts_cuda_ref_state.so is
the same reference library plus two accessors (oracle/ref_state_shim.cu) through which the worker
overwrites each reference session's state after its prompt (K/V rows, last hidden row, first token,
random state) with the state this library exported.  From equal state, and with this library in its
parity modes (SIMT projections, attention sums in the reference's order), every code and every next
token of every frame must be equal: test_frames_from_the_same_state.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIBRARY = os.path.join(ROOT, "oracle", "_ref", "libqwen3_tts_cuda_ref.so")
REF_STATE_LIBRARY = os.path.join(ROOT, "oracle", "_ref", "libqwen3_tts_cuda_ref_state.so")
WORKER = os.path.join(ROOT, "tests", "reference_frames_worker.py")


def run_worker(tmp, name, library, extra_env, extra_args=(), trace=True):
    out = os.path.join(tmp, name + ".json")
    stages = os.path.join(tmp, name + "_stages")
    env = dict(os.environ)
    env.update(extra_env)
    if trace:
        env["QWEN3_TTS_PARITY_TRACE"] = "1"
    if library is not None:
        env["QWEN3_TTS_TALKER_LIBRARY"] = library
    else:
        env.pop("QWEN3_TTS_TALKER_LIBRARY", None)
    proc = subprocess.run([sys.executable, WORKER, out, stages, *extra_args], env=env, capture_output=True,
                          text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    with open(out) as f:
        report = json.load(f)
    report["json_path"] = out
    # trace lines of the first prompt: everything up to and including the first "logits" line
    trace = []
    for line in proc.stderr.splitlines():
        if line.startswith("QWEN3_TTS_TRACE "):
            item = json.loads(line[len("QWEN3_TTS_TRACE "):])
            if item["stage"] == "float_logits":
                continue
            trace.append(item)
            if item["stage"] == "logits":
                break
    stage_tensors = {}
    for file in sorted(os.listdir(stages)):
        stage_tensors[file[:-5]] = np.fromfile(os.path.join(stages, file), dtype=np.uint16)
    return report, trace, stage_tensors


@pytest.fixture(scope="module")
def both(tmp_path_factory):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not os.path.exists(REF_LIBRARY):
        pytest.skip("oracle/_ref/libqwen3_tts_cuda_ref.so not built (needs a reference checkout)")
    tmp = str(tmp_path_factory.mktemp("reference_frames"))
    ref = run_worker(tmp, "reference", REF_LIBRARY, {"QWEN3_TTS_INT8_DECODE": "1", "QWEN3_TTS_STAGE_DUMP": "1"})
    # parity modes: the projection and attention kernels that keep the reference's summation order,
    # so that what differs is the composition and the prompt path, not the order of a sum
    os.makedirs(os.path.join(tmp, "ours_dump"), exist_ok=True)
    os.makedirs(os.path.join(tmp, "state"), exist_ok=True)
    ours = run_worker(tmp, "ours", None, {"QWEN3_TTS_STAGE_DUMP": os.path.join(tmp, "ours_dump/"),
                                          "Q3T_WORKER_GEMV_MODE": "0", "Q3T_WORKER_TC_MIN_ROWS": "65",
                                          "Q3T_WORKER_ATTENTION_MODE": "0"},
                      ("--export-state", os.path.join(tmp, "state")))
    return ref, ours


@pytest.fixture(scope="module")
def seeded(both, tmp_path_factory):
    """The reference's library started from this library's state after every prompt."""
    if not os.path.exists(REF_STATE_LIBRARY):
        pytest.skip("oracle/_ref/libqwen3_tts_cuda_ref_state.so not built (needs a reference checkout)")
    tmp = str(tmp_path_factory.mktemp("reference_seeded"))
    state_dir = os.path.join(os.path.dirname(both[1][0]["json_path"]), "state")
    ref = run_worker(tmp, "reference_seeded", REF_STATE_LIBRARY, {"QWEN3_TTS_INT8_DECODE": "1"},
                     ("--import-state", state_dir), trace=False)
    return ref[0], both[1][0]


def f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def ulp_distance(a, b):
    def ordered(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - (x & 0x7fff), x)
    return np.abs(ordered(a) - ordered(b))


def record(**fields):
    path = os.environ.get("Q3T_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(fields) + "\n")


def test_same_model_and_structure(both):
    (ref, _, _), (ours, _, _) = both
    assert ref["tensor_count"] == ours["tensor_count"] == 404
    assert ref["weight_bytes"] == ours["weight_bytes"] == 3_833_352_704
    assert len(ref["runs"]) == len(ours["runs"]) == 8
    for a, b in zip(ref["runs"], ours["runs"]):
        assert (a["prompt"], a["sessions"], a["sampled"]) == (b["prompt"], b["sessions"], b["sampled"])
        for sa, sb, fa, fb in zip(a["state"], b["state"], a["frames"], b["frames"]):
            if len(fa) == len(fb):
                assert sa[:3] == sb[:3], (a["prompt"], sa, sb)        # position, history count, frames generated
        for frames in b["frames"]:
            for codes in frames:
                assert len(codes) == 16 and all(0 <= c < 2048 for c in codes[1:]) and 0 <= codes[0] < 3072


def test_layer0_stages_of_the_prompt(both):
    """Same inputs, same weights: every layer-0 stage both libraries expose agrees to bf16 rounding."""
    (_, _, ref), (_, _, ours) = both
    shared = sorted(set(ref) & set(ours))
    assert {"input", "input_norm", "q_projection", "k_projection", "v_projection", "attention",
            "attention_residual", "gated_activation", "layer_output", "final_logits"} <= set(shared), shared
    summary = {}
    for name in shared:
        a, b = ref[name], ours[name]
        assert a.shape == b.shape, name
        d = ulp_distance(a, b)
        fa, fb = f32(a).astype(np.float64), f32(b).astype(np.float64)
        cosine = float(np.dot(fa, fb) / (np.linalg.norm(fa) * np.linalg.norm(fb) + 1e-30))
        summary[name] = {"exact": float((d == 0).mean()), "within_1": float((d <= 1).mean()),
                         "max_ulp": int(d.max()), "cosine": cosine}
    record(test="reference_layer0_stages", stages=summary)
    # the input row is gathered and projected before any difference in arithmetic can arise
    assert summary["input"]["within_1"] >= 0.999, summary["input"]
    # projections of an (almost) identical normalized row: rounding flips only
    for name in ("input_norm", "q_projection", "k_projection", "v_projection"):
        assert summary[name]["within_1"] >= 0.99 and summary[name]["cosine"] >= 0.99999, (name, summary[name])
    for name in ("attention", "attention_residual", "gated_activation", "layer_output"):
        assert summary[name]["cosine"] >= 0.9999, (name, summary[name])
    assert summary["final_logits"]["cosine"] >= 0.99, summary["final_logits"]


def test_prompt_trace_tracks_the_reference(both):
    """Per-layer statistics of the last prompt position through all 28 layers, the final norm and the
    largest logits, as both libraries print them."""
    (ref_report, ref_trace, _), (our_report, our_trace, _) = both
    keyed_ref = {(t["stage"], t.get("layer")): t for t in ref_trace}
    keyed_ours = {(t["stage"], t.get("layer")): t for t in our_trace}
    layers = [("layer", l) for l in range(28)]
    for key in [("input", -1)] + layers + [("final_norm", 28), ("logits", None)]:
        assert key in keyed_ref and key in keyed_ours, key
    drift = []
    for key in [("input", -1)] + layers + [("final_norm", 28)]:
        a, b = keyed_ref[key], keyed_ours[key]
        rms_gap = abs(a["rms"] - b["rms"]) / max(a["rms"], 1e-30)
        first_gap = float(np.max(np.abs(np.array(a["first"]) - np.array(b["first"]))) / max(a["rms"], 1e-30))
        drift.append({"stage": key[0], "layer": key[1], "rms_gap": rms_gap, "first16_gap_over_rms": first_gap})
        assert rms_gap <= 0.02, (key, a["rms"], b["rms"])
        assert first_gap <= 0.25, (key, first_gap)
    top_ref = [t["token"] for t in keyed_ref[("logits", None)]["top"]]
    top_ours = [t["token"] for t in keyed_ours[("logits", None)]["top"]]
    overlap = len(set(top_ref[:10]) & set(top_ours[:10]))
    record(test="reference_prompt_trace", drift=drift, top20_reference=top_ref, top20_ours=top_ours,
           first_token_reference=ref_report["prompt_first_token"], first_token_ours=our_report["prompt_first_token"])
    assert overlap >= 7, (top_ref, top_ours)
    assert our_report["prompt_first_token"] in top_ref[:3] and ref_report["prompt_first_token"] in top_ours[:3]


def test_frame_sequences_against_the_reference(both):
    """How far the code sequences of lockstep batches agree.  Every session of every run is compared
    frame by frame; the report keeps, per run, the number of sessions whose first token, first frame
    and whole sequence are identical and the first frame at which a session's codes differ."""
    (ref, _, _), (ours, _, _) = both
    rows = []
    for a, b in zip(ref["runs"], ours["runs"]):
        n = a["sessions"]
        same_first = sum(int(x == y) for x, y in zip(a["first_tokens"], b["first_tokens"]))
        first_frame_equal = whole_equal = 0
        diverged_at = []
        code_agreement = []
        for i in range(n):
            fa, fb = a["frames"][i], b["frames"][i]
            frames = min(len(fa), len(fb))
            at = next((f for f in range(frames) if fa[f] != fb[f]), None)
            diverged_at.append(at)
            first_frame_equal += int(frames > 0 and fa[0] == fb[0])
            whole_equal += int(at is None and a["next_tokens"][i] == b["next_tokens"][i])
            if frames:
                code_agreement.append(float(np.mean(np.array(fa[0]) == np.array(fb[0]))))
        rows.append({"prompt": a["prompt"], "sessions": n, "sampled": a["sampled"],
                     "same_first_token": same_first, "first_frame_equal": first_frame_equal,
                     "whole_sequence_equal": whole_equal, "first_divergent_frame": diverged_at,
                     "first_frame_code_agreement": float(np.mean(code_agreement)) if code_agreement else None})
    record(test="reference_frame_sequences", runs=rows)
    # Sessions of one batch share prompt and weights and differ in their seeds only: under greedy
    # decoding every session of a run must produce the same sequence, in both libraries.
    for run in ours["runs"] + ref["runs"]:
        if not run["sampled"]:
            for i in range(1, run["sessions"]):
                assert run["frames"][i] == run["frames"][0] and run["next_tokens"][i] == run["next_tokens"][0]
    # Across the two libraries nothing more is asserted here: each decodes from its own prompt's
    # cache, and with random weights the gap between the two largest logits is often smaller than
    # the rounding differences of the prompt paths, so first tokens and codes flip.  The frame
    # composition itself is pinned bit for bit by test_frames_from_the_same_state below.

def test_frames_from_the_same_state(seeded):
    """Frame composition proper.  The reference's sessions are handed this library's state after the
    prompt (K/V rows, last hidden row, first token, random state: oracle/ref_state_shim.cu), so the
    prompt paths no longer matter; from there both libraries run lockstep batches of 2 and 8 sessions
    through the same ABI calls, greedy and sampled.  In the parity modes (gemv mode 0, attention mode
    0, no tensor-core GEMM) every operator of the frame is bit-identical to the reference's kernel, so
    every code and every next token of every session must be equal."""
    ref, ours = seeded
    rows = []
    total = identical = first_frames = first_equal = 0
    for a, b in zip(ref["runs"], ours["runs"]):
        assert a["first_tokens"] == b["first_tokens"]
        n = a["sessions"]
        diverged_at = []
        for i in range(n):
            fa, fb = a["frames"][i], b["frames"][i]
            ta, tb = a["next_tokens"][i], b["next_tokens"][i]
            frames = min(len(fa), len(fb))
            at = next((f for f in range(frames) if fa[f] != fb[f] or ta[f] != tb[f]), None)
            diverged_at.append(at)
            total += 1
            identical += int(at is None and len(fa) == len(fb))
            if frames:
                first_frames += 1
                first_equal += int(fa[0] == fb[0] and ta[0] == tb[0])
        rows.append({"prompt": a["prompt"], "sessions": n, "sampled": a["sampled"],
                     "frames": [len(f) for f in b["frames"]], "first_divergent_frame": diverged_at,
                     "session0_reference": [a["frames"][0][:2], a["next_tokens"][0][:2]],
                     "session0_ours": [b["frames"][0][:2], b["next_tokens"][0][:2]]})
    record(test="reference_frames_from_same_state", runs=rows, sessions=total, identical_sequences=identical,
           first_frames=first_frames, first_frames_identical=first_equal)
    assert first_frames > 0
    assert first_equal == first_frames, rows
    assert identical == total, rows
