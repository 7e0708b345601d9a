#!/bin/bash
# Builds the reference's CUDA walker for sm_100 from its own sources where they lie
# (the read-only checkout named by FW_REFERENCE_DIR, see the default below) plus the harness
# and the gflags stand-in of this folder.
# Output only into oracle/_ref/ (kept out of git; it ships with the tree like the built library).  Flags follow the
# reference's CMakeLists.txt:28-49 (-O3 -lineinfo -maxrregcount=32, relocatable device code).
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${FW_REFERENCE_DIR:-/root/reference}"
[ -d "$REF/src" ] || { echo "reference sources not found at $REF"; exit 0; }
mkdir -p "$HERE/_ref"
OUT="$HERE/_ref/ref_walk"
if [ -x "$OUT" ] && [ "$OUT" -nt "$HERE/ref_harness.cu" ] && [ "$OUT" -nt "$HERE/ref_shim/gflags/gflags.h" ]; then
  echo "$OUT is up to date"; exit 0
fi
unset CC CXX
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
"$NVCC" -std=c++17 -O3 -lineinfo -maxrregcount=32 -rdc=true -arch=sm_100 -w \
  -Xcompiler -fopenmp -I"$HERE/ref_shim" -I"$REF/include" \
  "$HERE/ref_harness.cu" "$REF/src/walk.cu" "$REF/src/util.cu" \
  -o "$OUT" -lcurand -lcudadevrt -lgomp
echo "built $OUT"
