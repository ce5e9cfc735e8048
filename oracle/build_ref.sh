#!/usr/bin/env bash
# Builds oracle/_ref/ref_harness: the UNMODIFIED-in-behaviour GradCraft CPU path (CPUBackend +
# OpenBLAS cblas_sgemm + the naive nodes) driven by oracle/ref_harness.cpp.
#
# The reference ships for MSVC only, so a scratch copy of its headers (never committed, never
# placed in this repository) receives four mechanical portability patches before g++ sees it:
#   1. constructor template-ids (`AddNode<T>(...)`)            -> plain constructor names
#   2. constrained friend templates that GCC treats as new overloads -> members made public
#   3. `std::sqrtf`                                             -> `sqrtf`
#   4. `<corecrt_malloc.h>` / `<cblas.h>`                       -> two shim headers
# None of the patches touches arithmetic.  Outputs go to oracle/_ref/ only.
#
# Usage: oracle/build_ref.sh [reference_root]     (default: $GRADC_REFERENCE_ROOT, else a `reference` directory beside this repository)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${GRADC_REFERENCE_ROOT:-$HERE/../../reference}}"
OUT="$HERE/_ref"
if [ ! -d "$REF/gradc" ]; then
  echo "build_ref: reference tree not found at $REF (prebuilt oracle/_ref is used as is)"; exit 0
fi
SCRATCH="$(mktemp -d /tmp/gradc_ref_build.XXXXXX)"
trap 'rm -rf "$SCRATCH"' EXIT
mkdir -p "$OUT" "$SCRATCH/shim" "$SCRATCH/ref"
cp -r "$REF/gradc" "$SCRATCH/ref/gradc"
chmod -R u+w "$SCRATCH/ref"

# --- shim headers -----------------------------------------------------------------------------
cat > "$SCRATCH/shim/corecrt_malloc.h" <<'H'
#pragma once
#include <cstdlib>
static inline void* _aligned_malloc(size_t bytes, size_t align) {
    void* p = nullptr; if (bytes == 0) bytes = align;
    return posix_memalign(&p, align, bytes) == 0 ? p : nullptr; }
static inline void _aligned_free(void* p) { free(p); }
H
cat > "$SCRATCH/shim/cblas.h" <<'H'
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
typedef int blasint;
typedef enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_ORDER;
typedef enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
void cblas_sgemm(CBLAS_ORDER, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, blasint M, blasint N, blasint K, float alpha,
                 const float* A, blasint lda, const float* B, blasint ldb, float beta, float* C, blasint ldc);
void cblas_dgemm(CBLAS_ORDER, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, blasint M, blasint N, blasint K, double alpha,
                 const double* A, blasint lda, const double* B, blasint ldb, double beta, double* C, blasint ldc);
void openblas_set_num_threads(int);
int openblas_get_num_threads(void);
#ifdef __cplusplus
}
#endif
H

# --- portability patches ----------------------------------------------------------------------
G="$SCRATCH/ref/gradc"
sed -i -E 's/^(\s*)(AddNode|SubNode|MulNode|DivNode|NormalMatMulNode|BatchedMatMulNode)<T>\(/\1\2(/' "$G/graph/nodes/math_nodes.hpp"
# friend operator/matmul/blas-meta templates: drop the declarations, open the members instead
python3 - "$G/core/tensor.hpp" <<'PY'
import re, sys
p = sys.argv[1]
lines = open(p).read().split("\n")
out = []
for l in lines:
    st = l.strip()
    is_friend_fn = "friend" in st and "(" in st and "friend class" not in st
    if is_friend_fn:
        # drop the declaration and the template/requires header lines that belong to it
        if not st.startswith("template"):
            while out and (out[-1].strip().startswith("template <") or out[-1].strip().startswith("requires")):
                out.pop()
        continue
    out.append(l)
s = "\n".join(out)
s = s.replace("        private:\n            std::vector<int64_t> m_shape;", "        public:\n            std::vector<int64_t> m_shape;", 1)
open(p, "w").write(s)
PY
sed -i 's/std::sqrtf/sqrtf/g' "$G/backend/cuda/math_functors.cuh"

OPENBLAS="$(python3 - <<'PY'
import glob, sysconfig, os
sp = sysconfig.get_paths()["purelib"]
c = sorted(glob.glob(os.path.join(sp, "opencv_python_headless.libs", "libopenblas*.so*")))
print(c[0] if c else "")
PY
)"
CXXFLAGS="-std=c++23 -O2 -fopenmp -w -I$SCRATCH/shim -I$SCRATCH/ref -I/usr/local/cuda/include"
if [ -n "$OPENBLAS" ]; then
  BLASDIR="$(dirname "$OPENBLAS")"
  echo "build_ref: OpenBLAS = $OPENBLAS"
  g++ $CXXFLAGS "$HERE/ref_harness.cpp" -o "$OUT/ref_harness" \
      "$OPENBLAS" -Wl,--disable-new-dtags -Wl,-rpath,"$BLASDIR" -Wl,--allow-shlib-undefined \
      -L/usr/local/cuda/lib64 -lcudart -Wl,-rpath,/usr/local/cuda/lib64 \
      -Wl,--unresolved-symbols=ignore-all -fopenmp
  echo "openblas" > "$OUT/blas_kind.txt"
else
  echo "build_ref: no OpenBLAS found; linking the plain triple-loop sgemm in oracle/naive_cblas.c"
  gcc -O3 -march=native -fopenmp -c "$HERE/naive_cblas.c" -o "$SCRATCH/naive_cblas.o"
  g++ $CXXFLAGS "$HERE/ref_harness.cpp" "$SCRATCH/naive_cblas.o" -o "$OUT/ref_harness" \
      -L/usr/local/cuda/lib64 -lcudart -Wl,-rpath,/usr/local/cuda/lib64 \
      -Wl,--unresolved-symbols=ignore-all -fopenmp
  echo "naive" > "$OUT/blas_kind.txt"
fi
echo "build_ref: wrote $OUT/ref_harness"

# --- the reference's CUDA path (its two .cu files, nvcc for sm_100a, the flags of its own CMakeLists.txt:40) -------------
# A fifth portability patch, for nvcc on LP64: atomicMax / atomicMin have no `long*` overload, so the int64 instantiation
# of the reduction functors casts to `long long*` (same width, same operation).  Skipped when nvcc is absent.
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
if [ -x "$NVCC" ] && [ "${REF_SKIP_CUDA:-0}" != "1" ]; then
  python3 - "$G/backend/cuda/math_functors.cuh" <<'PY'
import sys
p = sys.argv[1]
s = open(p).read()
s = s.replace("atomicMax(adress, val);", "if constexpr (sizeof(T) == 8) atomicMax((long long*)adress, (long long)val); else atomicMax(adress, val);")
s = s.replace("atomicMin(adress, val);", "if constexpr (sizeof(T) == 8) atomicMin((long long*)adress, (long long)val); else atomicMin(adress, val);")
open(p, "w").write(s)
PY
  # the .cu files see lobotomized_broadcast_view() only through the friend declaration that patch 2 removes: pre-include its header
  NVFLAGS="-std=c++20 -gencode arch=compute_100a,code=sm_100a -O3 -use_fast_math -w -I$SCRATCH/shim -I$SCRATCH/ref -include $G/core/detail/tensor_lob_view.hpp"
  "$NVCC" $NVFLAGS -c "$G/backend/cuda/kernels_math.cu" -o "$SCRATCH/kernels_math.o" &
  "$NVCC" $NVFLAGS -c "$G/backend/cuda/kernels_utils.cu" -o "$SCRATCH/kernels_utils.o" &
  wait
  if [ -f "$SCRATCH/kernels_math.o" ] && [ -f "$SCRATCH/kernels_utils.o" ] && [ -n "$OPENBLAS" ]; then
    g++ $CXXFLAGS "$HERE/ref_harness.cpp" "$SCRATCH/kernels_math.o" "$SCRATCH/kernels_utils.o" -o "$OUT/ref_harness_cuda" \
        "$OPENBLAS" -Wl,--disable-new-dtags -Wl,-rpath,"$BLASDIR" -Wl,--allow-shlib-undefined \
        -L/usr/local/cuda/lib64 -lcudart -lcublas -lcurand -Wl,-rpath,/usr/local/cuda/lib64 -fopenmp
    echo "build_ref: wrote $OUT/ref_harness_cuda"
  else
    echo "build_ref: the reference's .cu files did not compile here; no ref_harness_cuda"
  fi
fi
