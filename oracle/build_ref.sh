#!/usr/bin/env bash
# Test infrastructure, not product code.
#
# Builds the UNMODIFIED reference math layer (engine/support/vmath.cu plus the two
# utility translation units it needs) into oracle/_ref/libkonan_ref.so, straight from
# the reference checkout, with the reference's own Release flags
# (engine/CMakeLists.txt:189-208: -fmad=false, -ffp-contract=off).  Only the host
# (device = -1) branch of each VMath function is ever called by the tests, so the
# library runs on machines without a GPU.  No reference source is copied: the
# compiler reads the files where they lie.
#
# usage: oracle/build_ref.sh [reference-root]   (default: $KONAN_REFERENCE)
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ref="${1:-${KONAN_REFERENCE:-}}"
[ -n "$ref" ] || { echo "usage: $0 <reference-root>  (or set KONAN_REFERENCE)" >&2; exit 2; }
eng="$ref/source/engine"
out="$here/_ref"
cuda="${CUDA_HOME:-/usr/local/cuda}"
[ -f "$eng/support/vmath.cu" ] || { echo "reference not found under $ref" >&2; exit 3; }
mkdir -p "$out"
"$cuda/bin/nvcc" -O3 -std=c++14 -DFOR_LINUX -fmad=false \
    -Xcompiler "-ffp-contract=off -fpermissive -fPIC -w" \
    -gencode arch=compute_100a,code=sm_100a \
    -c "$eng/support/vmath.cu" -o "$out/vmath.o"
for f in vexception vvalue; do
  g++ -O2 -std=c++14 -DFOR_LINUX -fPIC -fpermissive -ffp-contract=off -w \
      -I"$cuda/include" -c "$eng/utils/$f.cpp" -o "$out/$f.o"
done
g++ -shared -o "$out/libkonan_ref.so" "$out/vmath.o" "$out/vexception.o" "$out/vvalue.o" \
    -L"$cuda/lib64" -lcudart -Wl,--no-undefined
rm -f "$out"/*.o
echo "built $out/libkonan_ref.so"
