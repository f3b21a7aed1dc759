#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.  Links TensorPlay's own P10 core (objects from build_ref.sh, with its
# CUDA allocator switched on), the registration adapter of this repository and libtpb200.so into
# oracle/_ref/adapter_check, the C++-level check of the drop-in boundary (tests/adapter_check.cpp).
# Needs a TensorPlay checkout; skips quietly without one.  Nothing of the reference is copied.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(dirname "$HERE")"
REF="${TP_REFERENCE_ROOT:-}"
OUT="$HERE/_ref"
CUDA="${CUDA_HOME:-/usr/local/cuda}"
if [ -z "$REF" ] || [ ! -f "$REF/p10/src/backend/cuda/CUDAAllocator.cpp" ] || [ ! -d "$OUT/obj" ]; then
    echo "build_adapter_check: reference checkout or oracle/_ref/obj missing; skipping" >&2
    exit 0
fi
[ -f "$ROOT/tensorplay_b200/libtpb200.so" ] || { echo "build libtpb200.so first" >&2; exit 1; }
CXX="g++ -std=c++20 -O2 -w -fPIC -I$REF/p10/include -I$OUT/gen -I$CUDA/include"
mkdir -p "$OUT/obj_cuda"
$CXX -DUSE_CUDA -c "$REF/p10/src/Allocator.cpp" -o "$OUT/obj_cuda/Allocator.o"
$CXX -DUSE_CUDA -c "$REF/p10/src/backend/cuda/CUDAAllocator.cpp" -o "$OUT/obj_cuda/CUDAAllocator.o"
$CXX -c "$ROOT/tensorplay_b200/csrc/adapter/tensorplay_adapter.cpp" -o "$OUT/obj_cuda/adapter.o"
$CXX -c "$ROOT/tests/adapter_check.cpp" -o "$OUT/obj_cuda/adapter_check.o"
OBJS=$(ls "$OUT"/obj/*.o | grep -v '/Allocator.o$')
g++ -o "$OUT/adapter_check" "$OUT"/obj_cuda/*.o $OBJS -fopenmp \
    -L"$ROOT/tensorplay_b200" -ltpb200 -L"$HERE" -ltporacle -L"$CUDA/lib64" -lcudart \
    -Wl,-rpath,'$ORIGIN/../../tensorplay_b200' -Wl,-rpath,'$ORIGIN/..' -Wl,-rpath,"$CUDA/lib64"
echo "build_adapter_check: built $OUT/adapter_check"
