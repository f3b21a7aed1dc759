#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.  Builds oracle/_ref/tpx_check (tests/tpx_check.cpp): TensorPlay's autograd
# engine and generated backward nodes (tpx/src, the generator's TPXOpsGenerated.cpp), its P10 core and
# its own CUDA kernels for everything that is NOT a reduction (factory, view, copy, arithmetic,
# pointwise: compiled with nvcc from the sources where they lie), plus the registration adapter and
# libtpb200.so of this repository.  The reference's ReductionKernels.cu is not built: reductions on
# CUDA tensors can only come from the new kernels.  Needs TP_REFERENCE_ROOT (a TensorPlay checkout)
# and the objects of build_ref.sh / build_adapter_check.sh; skips quietly without them.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(dirname "$HERE")"
REF="${TP_REFERENCE_ROOT:-}"
OUT="$HERE/_ref"
CUDA="${CUDA_HOME:-/usr/local/cuda}"
if [ -z "$REF" ] || [ ! -d "$REF/tpx/src" ] || [ ! -f "$OUT/obj_cuda/adapter.o" ]; then
    echo "build_tpx_check: reference checkout or oracle/_ref/obj_cuda missing; skipping" >&2
    exit 0
fi
if [ -f "$OUT/tpx_check" ] && [ "$OUT/tpx_check" -nt "$ROOT/tests/tpx_check.cpp" ] && [ "$OUT/tpx_check" -nt "$OUT/obj_cuda/adapter.o" ] \
   && [ "$OUT/tpx_check" -nt "$ROOT/tensorplay_b200/libtpb200.so" ] && [ "${1:-}" != "--force" ]; then
    echo "build_tpx_check: $OUT/tpx_check is up to date"
    exit 0
fi
mkdir -p "$OUT/obj_tpx"
INC="-I$REF/p10/include -I$REF/tpx/include -I$OUT/gen -I$CUDA/include"
NVCC="$CUDA/bin/nvcc -std=c++17 -gencode arch=compute_100a,code=sm_100a -DUSE_CUDA -DUSE_CUDNN -w -Xcompiler -fPIC $INC -I$REF/p10/src/backend/cuda -I/usr/include/x86_64-linux-gnu"
CXX="g++ -std=c++20 -O2 -w -fPIC -DUSE_CUDA -DUSE_CUDNN $INC -I$REF/p10/src/backend/cuda"
pids=()
for f in Factory View Copy Arithmetic Pointwise; do
    [ -f "$OUT/obj_tpx/cuda_$f.o" ] || { $NVCC -c "$REF/p10/src/backend/cuda/${f}Kernels.cu" -o "$OUT/obj_tpx/cuda_$f.o" & pids+=($!); }
done
for f in Autograd AutogradMetaInterface Engine Tensor; do
    $CXX -c "$REF/tpx/src/$f.cpp" -o "$OUT/obj_tpx/tpx_$f.o" & pids+=($!)
done
$CXX -c "$OUT/gen/tensorplay/ops/TPXOpsGenerated.cpp" -o "$OUT/obj_tpx/tpx_ops.o" & pids+=($!)
$CXX -c "$REF/p10/src/backend/cuda/CUDAContext.cpp" -o "$OUT/obj_tpx/CUDAContext.o" & pids+=($!)
$CXX -c "$ROOT/tests/tpx_check.cpp" -o "$OUT/obj_tpx/tpx_check.o" & pids+=($!)
for p in "${pids[@]}"; do wait "$p"; done
OBJS=$(ls "$OUT"/obj/*.o | grep -v '/Allocator.o$')
g++ -o "$OUT/tpx_check" "$OUT"/obj_tpx/*.o "$OUT/obj_cuda/Allocator.o" "$OUT/obj_cuda/CUDAAllocator.o" "$OUT/obj_cuda/adapter.o" $OBJS -fopenmp \
    -L"$ROOT/tensorplay_b200" -ltpb200 -L"$CUDA/lib64" -lcudart -lcublas -lcurand -lcudnn \
    -Wl,-rpath,'$ORIGIN/../../tensorplay_b200' -Wl,-rpath,"$CUDA/lib64"
echo "build_tpx_check: built $OUT/tpx_check"
