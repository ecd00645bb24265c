"""Worker of tests/test_gpu_reference_frames.py: drives ONE build of the native talker C ABI through a
fixed scenario and writes what it observed to a JSON file.  Run as a subprocess, once with this
repository's library and once with the reference project's own library compiled for sm_100a
(oracle/_ref/libqwen3_tts_cuda_ref.so, int8 decode switched on), so that the two never share a
process, an environment or a CUDA context:

    QWEN3_TTS_TALKER_LIBRARY=<lib.so> python tests/reference_frames_worker.py <out.json> <stage dir> \
        [--export-state DIR | --import-state DIR]

Both libraries get the same 404 synthetic tensors whose decode matrices are exactly
int8-representable (synth.make_tensor(exact_int8=True)), the same prompts, seeds and sampling
configurations, and are called through the same functions of the reference's ABI only:
model_create / upload_tensor / finalize, session_create / prefill, model_batch_next_frame_begin_v2 /
session_next_frame_finish_v2.  Frame codes are read from the device buffer the ABI hands out.
The parity hooks (QWEN3_TTS_PARITY_TRACE lines on stderr, QWEN3_TTS_STAGE_DUMP files) are switched
on by the parent; the stage files of the first prompt are copied into <stage dir>.

--export-state DIR (this repository's library): after the prompts of a run, every session's state
is written to DIR/run<k>.npz: the K and V rows of the prompt in all 28 layers, the last hidden row,
the first semantic token and the sampler's random state.
--import-state DIR (oracle/_ref/libqwen3_tts_cuda_ref_state.so, the reference's library plus the two
accessors of oracle/ref_state_shim.cu): after its own prompts, every session's state is overwritten
with the exported one, so that both libraries start the first frame from the same bits.
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

FRAMES = 8
PROMPT_LENGTH = 24


def prompts():
    rng = np.random.default_rng(2024)
    text = [int(t) for t in rng.integers(0, 151936, size=PROMPT_LENGTH)]
    codec = [-1] * PROMPT_LENGTH
    for i in range(3, PROMPT_LENGTH, 5):
        codec[i] = int(rng.integers(0, 3072))      # positions with text and codec input
    text[7], codec[7] = -1, 2149                   # a position with codec input only
    return {"long": (text, codec), "short": (text[:1], [-1])}


class RefSessionState(C.Structure):
    """Q3tRefSessionState of oracle/ref_state_shim.cu."""
    _fields_ = [("keys", C.c_void_p * 28), ("values", C.c_void_p * 28), ("last_hidden", C.c_void_p),
                ("semantic_history", C.c_void_p), ("random_state", C.c_void_p), ("sampled_token", C.c_void_p),
                ("position", C.c_int32),
                ("history_count", C.c_int32), ("max_sequence_length", C.c_int32),
                ("current_token", C.c_uint32), ("phase", C.c_uint32)]


def main() -> None:
    out_path, stage_dir = sys.argv[1], sys.argv[2]
    export_dir = sys.argv[4] if len(sys.argv) > 4 and sys.argv[3] == "--export-state" else None
    import_dir = sys.argv[4] if len(sys.argv) > 4 and sys.argv[3] == "--import-state" else None
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

    def to_device(pointer, array):
        array = np.ascontiguousarray(array)
        rc = cudart.cudaMemcpy(C.c_void_p(pointer), array.ctypes.data_as(C.c_void_p), array.nbytes, 1)
        if rc != 0:
            raise RuntimeError(f"cudaMemcpy returned {rc}")

    def export_state(path, sessions, prompt_length):
        fields = {}
        for i, x in enumerate(sessions):
            hidden, _, rng = x.read_state()
            kv = [x.read_kv(layer, 0, prompt_length) for layer in range(28)]
            fields[f"keys{i}"] = np.stack([k for k, _ in kv])
            fields[f"values{i}"] = np.stack([v for _, v in kv])
            fields[f"hidden{i}"] = hidden
            fields[f"scalars{i}"] = np.array([rng, int(x.current_semantic_token)], dtype=np.uint64)
        np.savez(path, **fields)

    def import_state(path, sessions, prompt_length):
        lib = native.library()
        lib.q3t_ref_session_state.argtypes = [C.c_void_p, C.POINTER(RefSessionState)]
        lib.q3t_ref_session_set_current_token.argtypes = [C.c_void_p, C.c_uint32]
        data = np.load(path)
        for i, x in enumerate(sessions):
            st = RefSessionState()
            if lib.q3t_ref_session_state(x._handle, C.byref(st)) != 0:
                raise RuntimeError("q3t_ref_session_state failed")
            if st.position != prompt_length or st.history_count != 1:
                raise RuntimeError(f"unexpected reference state {st.position} {st.history_count}")
            for layer in range(28):
                to_device(st.keys[layer], data[f"keys{i}"][layer])
                to_device(st.values[layer], data[f"values{i}"][layer])
            to_device(st.last_hidden, data[f"hidden{i}"])
            rng, token = (int(v) for v in data[f"scalars{i}"])
            if token == 2150:          # this library's prompt ended the session at once: nothing to seed
                x.current_semantic_token, x.ended = token, True
                continue
            to_device(st.random_state, np.array([rng], dtype=np.uint64))
            to_device(st.semantic_history, np.array([token], dtype=np.int32))
            to_device(st.sampled_token, np.array([token], dtype=np.int32))
            if lib.q3t_ref_session_set_current_token(x._handle, token) != 0:
                raise RuntimeError("q3t_ref_session_set_current_token failed")
            x.current_semantic_token = token
            x.ended = False

    if hasattr(native.library(), "q3t_set_gemv_mode") and os.environ.get("Q3T_WORKER_GEMV_MODE"):
        native.set_gemv_mode(int(os.environ["Q3T_WORKER_GEMV_MODE"]))

    if hasattr(native.library(), "q3t_set_attention_mode") and os.environ.get("Q3T_WORKER_ATTENTION_MODE"):
        native.set_attention_mode(int(os.environ["Q3T_WORKER_ATTENTION_MODE"]))

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
    run_index = 0
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
                state_file = f"run{run_index}.npz"
                run_index += 1
                if export_dir:
                    export_state(os.path.join(export_dir, state_file), sessions, len(all_prompts[prompt_name][0]))
                if import_dir:
                    import_state(os.path.join(import_dir, state_file), sessions, len(all_prompts[prompt_name][0]))
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
