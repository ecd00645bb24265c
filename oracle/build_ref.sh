#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.
# Compiles the reference project's own CUDA code, from the sources where they lie
# in a checkout of luka-loehr/qwen3-tts-native, for sm_100a.  Three outputs in
# oracle/_ref/ (git-ignored):
#   libq3t_ref.so               its three kernel files linked with ref_shim.cu: the
#                               kernel launchers one by one, for operator parity;
#   libqwen3_tts_cuda_ref.so    its whole talker library (eight .cu files + cuBLAS)
#                               under its own C ABI: model, sessions and frames, for
#                               parity of the frame composition and the prompt path;
#   libqwen3_tts_cuda_ref_state.so  the same library with two more exports (ref_state_shim.cu)
#                               through which a test seeds a session's state after the prompt.
# No reference source is copied into this repository and its CMake build is
# bypassed (that build pins sm_121 and CUDA 13).
#
#   usage: oracle/build_ref.sh path/to/reference/checkout
#          (or QWEN3_TTS_REFERENCE_CHECKOUT=... oracle/build_ref.sh)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${QWEN3_TTS_REFERENCE_CHECKOUT:-}}"
if [ -z "$REF" ]; then
    echo "usage: $0 path/to/reference/checkout" >&2
    exit 2
fi
SRC="$REF/native/qwen3-tts-native/native"
if [ ! -f "$SRC/src/int8_gemv.cu" ]; then
    echo "reference checkout not found at $REF; nothing built" >&2
    exit 3
fi
OUT="$HERE/_ref"
mkdir -p "$OUT"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
"$NVCC" -std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a -shared -Xcompiler -fPIC \
    -I"$SRC/include" -I"$SRC/src" \
    "$SRC/src/int8_gemv.cu" "$SRC/src/talker_kernels.cu" "$SRC/src/sampling_kernels.cu" \
    "$HERE/ref_shim.cu" \
    -Xlinker -rpath -Xlinker /usr/local/cuda/lib64 \
    -o "$OUT/libq3t_ref.so"
echo "built $OUT/libq3t_ref.so"
"$NVCC" -std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a -shared -Xcompiler -fPIC \
    -I"$SRC/include" -I"$SRC/src" \
    "$SRC/src/gemv.cu" "$SRC/src/int8_gemv.cu" "$SRC/src/primitive_parity.cu" "$SRC/src/runtime.cu" \
    "$SRC/src/sampling_kernels.cu" "$SRC/src/talker.cu" "$SRC/src/talker_kernels.cu" "$SRC/src/weights.cu" \
    -lcublas -Xlinker -rpath -Xlinker /usr/local/cuda/lib64 \
    -o "$OUT/libqwen3_tts_cuda_ref.so"
echo "built $OUT/libqwen3_tts_cuda_ref.so"
# the same library with talker.cu compiled through ref_state_shim.cu (two more exports that let
# a test read and seed a session's state after the prompt)
"$NVCC" -std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a -shared -Xcompiler -fPIC \
    -I"$SRC/include" -I"$SRC/src" \
    "$SRC/src/gemv.cu" "$SRC/src/int8_gemv.cu" "$SRC/src/primitive_parity.cu" "$SRC/src/runtime.cu" \
    "$SRC/src/sampling_kernels.cu" "$HERE/ref_state_shim.cu" "$SRC/src/talker_kernels.cu" "$SRC/src/weights.cu" \
    -lcublas -Xlinker -rpath -Xlinker /usr/local/cuda/lib64 \
    -o "$OUT/libqwen3_tts_cuda_ref_state.so"
echo "built $OUT/libqwen3_tts_cuda_ref_state.so"
