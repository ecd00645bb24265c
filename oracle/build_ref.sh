#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.
# Compiles the reference project's own CUDA kernels, from the sources where they
# lie in a checkout of luka-loehr/qwen3-tts-native, for sm_100a and links them
# with ref_shim.cu into oracle/_ref/libq3t_ref.so.  No reference source is copied
# into this repository and its CMake build is bypassed (that build pins sm_121
# and CUDA 13).  The output directory is git-ignored.
#
#   usage: oracle/build_ref.sh [path/to/reference/checkout]
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-/root/reference}"
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
