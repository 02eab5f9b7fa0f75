#!/usr/bin/env bash
# Test infrastructure, not product code.
#
# Compiles the drop-in stub (matmul_kernel_stub.cpp) together with a small C harness against the reference's own
# headers and links it to aakaar_b200/lib/libakr_b200.so. Output: oracle/_ref/libakr_dropin.so (git-ignored; it
# travels to the GPU box like the other prebuilt checkers). No reference source is copied into this repository.
#
#   usage: oracle/integration/build_stub.sh [reference_root]   (or AAKAAR_REFERENCE=...)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(cd "$HERE/../.." && pwd)"
REF="${1:-${AAKAAR_REFERENCE:-/root/reference}}"
OUT="$ROOT/oracle/_ref"
if [ ! -d "$REF/src" ]; then
  echo "build_stub: no reference checkout at $REF (keeping any prebuilt $OUT/libakr_dropin.so)"; exit 0
fi
if [ ! -f "$ROOT/aakaar_b200/lib/libakr_b200.so" ]; then
  echo "build_stub: aakaar_b200/lib/libakr_b200.so is not built yet"; exit 1
fi
PY="${PYTHON:-python}"
PYINC="$($PY -c 'import sysconfig; print(sysconfig.get_paths()["include"])')"
PBINC="$($PY -c 'import pybind11; print(pybind11.get_include())')"
CUDA="${CUDA_HOME:-/usr/local/cuda}"
mkdir -p "$OUT"
TARGET="$OUT/libakr_dropin.so"
if [ -f "$TARGET" ] && [ "$TARGET" -nt "$HERE/matmul_kernel_stub.cpp" ] && [ "$TARGET" -nt "$HERE/stub_harness.cpp" ] \
   && [ "$TARGET" -nt "$ROOT/include/akr_b200.h" ] && [ "$TARGET" -nt "$REF/src/tensor.h" ]; then
  echo "build_stub: $TARGET is up to date"; exit 0
fi
g++ -O1 -std=c++17 -fPIC -shared -w -I"$REF/src" -I"$ROOT/include" -I"$PYINC" -I"$PBINC" -I"$CUDA/include" \
    "$HERE/matmul_kernel_stub.cpp" "$HERE/stub_harness.cpp" -o "$TARGET" \
    -L"$ROOT/aakaar_b200/lib" -lakr_b200 -L"$CUDA/lib64" -lcudart \
    -Wl,--disable-new-dtags -Wl,-rpath,'$ORIGIN/../../aakaar_b200/lib' -Wl,-rpath,"$CUDA/lib64"
echo "build_stub: built $TARGET"
