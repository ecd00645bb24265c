"""Worker of tests/test_gpu_reference_frames.py: drives ONE build of the native talker C ABI through a
fixed scenario and writes what it observed to a JSON file.  Run as a subprocess, once with this
repository's library and once with the reference project's own library compiled for sm_100a
(oracle/_ref/libqwen3_tts_cuda_ref.so, int8 decode switched on), so that the two never share a
process, an environment or a CUDA context:

    QWEN3_TTS_TALKER_LIBRARY=<lib.so> python tests/reference_frames_worker.py <out.json> <stage dir>

Both libraries get the same 404 synthetic tensors whose decode matrices are exactly
int8-representable (synth.make_tensor(exact_int8=True)), the same prompts, seeds and sampling
configurations, and are called through the same functions of the reference's ABI only:
model_create / upload_tensor / finalize, session_create / prefill, model_batch_next_frame_begin_v2 /
session_next_frame_finish_v2.  Frame codes are read from the device buffer the ABI hands out.
The parity hooks (QWEN3_TTS_PARITY_TRACE lines on stderr, QWEN3_TTS_STAGE_DUMP files) are switched
on by the parent; the stage files of the first prompt are copied into <stage dir>.
"""
from __future__ import annotations

import ctypes as C
import importlib
import json
import os
import shutil
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FRAMES = 6
PROMPT_LENGTH = 24


def prompts():
    rng = np.random.default_rng(2024)
    text = [int(t) for t in rng.integers(0, 151936, size=PROMPT_LENGTH)]
    codec = [-1] * PROMPT_LENGTH
    for i in range(3, PROMPT_LENGTH, 5):
        codec[i] = int(rng.integers(0, 3072))      # positions with text and codec input
    text[7], codec[7] = -1, 2149                   # a position with codec input only
    return {"long": (text, codec), "short": (text[:1], [-1])}


def main() -> None:
    out_path, stage_dir = sys.argv[1], sys.argv[2]
    import torch
    torch.cuda.set_device(0)
    q3t = importlib.import_module("qwen3-tts-native_b200")
    synth = importlib.import_module("qwen3-tts-native_b200.synth")
    native = q3t.native
    cudart = C.CDLL("libcudart.so.12")

    def device_codes(pending):
        host = (C.c_uint16 * 16)()
        rc = cudart.cudaMemcpy(host, C.c_void_p(pending.device_codes), 32, 2)      # device to host
        if rc != 0:
            raise RuntimeError(f"cudaMemcpy returned {rc}")
        return [int(c) for c in host]

    if hasattr(native.library(), "q3t_set_gemv_mode") and os.environ.get("Q3T_WORKER_GEMV_MODE"):
        native.set_gemv_mode(int(os.environ["Q3T_WORKER_GEMV_MODE"]))

    model = q3t.NativeTalkerModel.load(0, synth.checkpoint(seed=0, exact_int8=True))
    if os.environ.get("Q3T_WORKER_TC_MIN_ROWS"):
        model.set_option("tc_min_rows", int(os.environ["Q3T_WORKER_TC_MIN_ROWS"]))
    report = {"library": os.environ.get("QWEN3_TTS_TALKER_LIBRARY", "default"),
              "tensor_count": int(model.memory.tensor_count),
              "weight_bytes": int(model.memory.shared_weight_bytes), "runs": []}
    greedy = q3t.SamplingConfig.greedy()
    talker = q3t.SamplingConfig(True, 50, 1.0, 0.9, 1.05)
    predictor = q3t.SamplingConfig(True, 50, 1.0, 0.9, 1.0)
    all_prompts = prompts()

    # ---- the prompt path alone: one session, the long prompt, greedy first token; hooks observe it
    os.makedirs(stage_dir, exist_ok=True)
    default_stage_dir = "/tmp/native_stages"
    os.makedirs(default_stage_dir, exist_ok=True)
    s = model.start_prompt(*all_prompts["long"], 64, 11, greedy, greedy)
    report["prompt_first_token"] = int(s.current_semantic_token)
    s.close()
    source = os.environ.get("QWEN3_TTS_STAGE_DUMP", "")
    source = source if "/" in source else default_stage_dir
    for name in sorted(os.listdir(source)):
        if name.endswith(".bf16") and os.path.abspath(source) != os.path.abspath(stage_dir):
            shutil.copy(os.path.join(source, name), os.path.join(stage_dir, name))

    # ---- frames: lockstep batches of 2 and 8 sessions, short and long prompts, greedy and sampled
    for prompt_name in ("short", "long"):
        for n in (2, 8):
            for sampled in (False, True):
                tcfg, pcfg = (talker, predictor) if sampled else (greedy, greedy)
                sessions = [model.start_prompt(*all_prompts[prompt_name], 64, 100 + i, tcfg, pcfg)
                            for i in range(n)]
                run = {"prompt": prompt_name, "sessions": n, "sampled": sampled,
                       "first_tokens": [int(x.current_semantic_token) for x in sessions],
                       "frames": [[] for _ in range(n)], "next_tokens": [[] for _ in range(n)]}
                live = list(range(n))
                for f in range(FRAMES):
                    live = [i for i in live if not sessions[i].ended]
                    if len(live) < 2:
                        break
                    pending = model.batch_begin_device_frames([sessions[i] for i in live], [7000 + f] * len(live))
                    for i, p in zip(live, pending):
                        frame = p.finish_without_consumer()
                        run["frames"][i].append(device_codes(p))
                        run["next_tokens"][i].append(int(frame.next_semantic_token))
                states = [x.runtime_state() for x in sessions]
                run["state"] = [[st.talker_position, st.semantic_history_count, st.frames_generated,
                                 st.device_sample_count] for st in states]
                report["runs"].append(run)
                for x in sessions:
                    x.close()
    model.close()
    with open(out_path, "w") as f:
        json.dump(report, f)


if __name__ == "__main__":
    main()
