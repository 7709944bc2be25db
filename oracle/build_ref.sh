#!/usr/bin/env bash
# Builds the UNMODIFIED reference sporder library (CUDA) for sm_100a from the
# sources where they lie in the reference checkout, plus a small shim that
# exposes the reference's internal csg top-k table.  Outputs go only to
# oracle/_ref/ (git-ignored).  The result needs a GPU to run: it is used by the
# GPU parity tests and by bench.py as the "reference CUDA build on this box"
# comparison, never by the product path.
#
# usage: oracle/build_ref.sh <reference_root>   (or SPORDER_REFERENCE_ROOT in the environment)
set -euo pipefail
REF="${1:-${SPORDER_REFERENCE_ROOT:-}}"
if [ -z "$REF" ]; then
  echo "build_ref: no reference checkout named (argument or SPORDER_REFERENCE_ROOT); keeping prebuilt files" >&2
  exit 0
fi
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
SP="$REF/sporder"
if [ ! -d "$SP/src" ]; then
  echo "build_ref: reference sources not found under $REF; keeping prebuilt files" >&2
  exit 0
fi
mkdir -p "$OUT"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
FLAGS=(-std=c++20 -gencode arch=compute_100a,code=sm_100a --expt-relaxed-constexpr
       --ftz=true --extra-device-vectorization -lineinfo -O3 -Xcompiler -fPIC
       -I "$SP/include" -I "$SP/src")
SRCS=("$SP"/src/sporder.cpp "$SP"/src/*.cu "$SP"/src/common/*.cu "$SP"/src/csg/*.cu
      "$SP"/src/cg/*.cu "$SP"/src/hm/*.cu)
"$NVCC" "${FLAGS[@]}" -shared -o "$OUT/libsporder_ref.so" "${SRCS[@]}" "$HERE/ref_shim.cu" \
        -lcusparse -lcurand
echo "build_ref: wrote $OUT/libsporder_ref.so"
