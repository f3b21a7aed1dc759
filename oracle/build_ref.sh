#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.  Compiles the reference's own CPU reduction path, from the sources
# where they lie in a TensorPlay checkout, into oracle/_ref/libtpref.so (binaries only; no
# reference source is copied into this repository).  The result is used to validate the C
# restatement in oracle/tp_oracle.c and as the timed CPU baseline.
#
# What it runs:
#   1. the reference's generator  tools/codegen/gen.py  on its two yaml files -- the CPU kernels
#      call generated Tensor methods (Tensor::mean, operator-, ...), so TensorGenerated.{h,cpp}
#      is needed; only PyYAML is required.  The schema gets one additive entry (top-k, which the
#      reference does not declare: tensorplay_b200/csrc/adapter/topk_schema.yaml), so that the
#      generated Tensor class has the topk method the adapter check calls, and the derivatives get
#      additive formulas for the dim variants of sum / mean / var / std
#      (tensorplay_b200/csrc/adapter/derivatives_add.yaml), which the autograd check uses;
#   2. g++ with the reference's own flags (CMakeLists.txt:213,470: -O3 -march=native, OpenMP on,
#      no USE_CUDA / USE_ONEDNN / USE_MKL) on the P10 core and CPU kernel files;
#   3. a link with oracle/ref_driver.cpp.
# The reference's CMake build is not run.  TP_REFERENCE_ROOT names the checkout; without it the
# script skips quietly (exit 0) and whatever was built before stays in place.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${TP_REFERENCE_ROOT:-}"
OUT="$HERE/_ref"
SCHEMA_ADD="$HERE/../tensorplay_b200/csrc/adapter/topk_schema.yaml"
DERIV_ADD="$HERE/../tensorplay_b200/csrc/adapter/derivatives_add.yaml"
if [ -z "$REF" ] || [ ! -f "$REF/p10/src/backend/cpu/ReductionKernels.cpp" ]; then
    echo "build_ref: TP_REFERENCE_ROOT does not name a TensorPlay checkout; skipping" >&2
    exit 0
fi
if [ -f "$OUT/libtpref.so" ] && [ "$OUT/libtpref.so" -nt "$HERE/ref_driver.cpp" ] && [ "$OUT/libtpref.so" -nt "$SCHEMA_ADD" ] && [ "$OUT/libtpref.so" -nt "$DERIV_ADD" ] && [ "${1:-}" != "--force" ]; then
    echo "build_ref: $OUT/libtpref.so is up to date"
    exit 0
fi
mkdir -p "$OUT/gen/tensorplay/ops" "$OUT/obj"
PKG_SCRATCH="$(mktemp -d)"       # the generator also writes Python stubs; they are not needed
trap 'rm -rf "$PKG_SCRATCH"' EXIT
# the reference's schema plus the one additive entry for top-k (the reference declares none)
cat "$REF/config/native_functions.yaml" > "$OUT/native_functions_plus_topk.yaml"
printf '\n' >> "$OUT/native_functions_plus_topk.yaml"
grep -v '^#' "$SCHEMA_ADD" >> "$OUT/native_functions_plus_topk.yaml"
# ... and its derivatives plus the additive formulas for the dim variants of the reductions
cat "$REF/config/derivatives.yaml" > "$OUT/derivatives_plus_dims.yaml"
printf '\n' >> "$OUT/derivatives_plus_dims.yaml"
grep -v '^#' "$DERIV_ADD" >> "$OUT/derivatives_plus_dims.yaml"
python3 "$REF/tools/codegen/gen.py" --yaml "$OUT/native_functions_plus_topk.yaml" \
    --derivatives "$OUT/derivatives_plus_dims.yaml" --out_dir "$OUT/gen/tensorplay/ops" \
    --pkg_out "$PKG_SCRATCH" > "$OUT/gen.log" 2>&1

CXXFLAGS="-std=c++20 -O3 -march=native -fopenmp -w -fPIC -I$REF/p10/include -I$OUT/gen"
SRCS=()
for f in Allocator Device Dispatcher Exception Generator Scalar SizesAndStrides Stacktrace TensorImpl OneDNNContext Tensor; do
    SRCS+=("$REF/p10/src/$f.cpp")
done
for f in Arithmetic Comparison Copy Factory Pointwise Random Reduction View; do
    SRCS+=("$REF/p10/src/backend/cpu/${f}Kernels.cpp")
done
SRCS+=("$OUT/gen/tensorplay/ops/TensorGenerated.cpp")

compile_one() {
    src="$1"; base="$(basename "${src%.cpp}")"
    case "$src" in */backend/cpu/*) base="cpu_$base";; esac
    g++ $CXXFLAGS -c "$src" -o "$OUT/obj/$base.o"
}
export -f compile_one
export CXXFLAGS OUT
printf '%s\n' "${SRCS[@]}" | xargs -P "$(nproc)" -I{} bash -c 'compile_one "$@"' _ {}

g++ $CXXFLAGS -shared -o "$OUT/libtpref.so" "$HERE/ref_driver.cpp" "$OUT"/obj/*.o -fopenmp
echo "build_ref: built $OUT/libtpref.so"
