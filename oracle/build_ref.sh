#!/bin/sh
# Builds the REFERENCE's own seblas kernels for sm_100a, from the sources where they lie in the reference tree,
# together with oracle/ref/ref_shim.cu, into oracle/_ref/libseblas_ref.so (git-ignored). No reference source is
# copied: the one unportable header (seio/logging/LogUtils.cuh -> <windows.h>) is skipped by predefining its
# include guard and force-including oracle/ref/log_stub.h.
# Usage: oracle/build_ref.sh [reference_root]   (default: where the reference tree is mounted, see REF below)
set -e
REF="${1:-/root/reference}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
if [ ! -d "$REF/seblas" ]; then
    echo "build_ref: $REF/seblas not found (the reference tree is not mounted); keeping any prebuilt library" >&2
    exit 0
fi
mkdir -p "$OUT/obj"
NVCC="${NVCC:-nvcc}"
FLAGS="-std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -Xcompiler -fPIC -w -DCRUSADER_LOGUTILS_CUH -include $HERE/ref/log_stub.h -I/usr/include/x86_64-linux-gnu -I$REF"
pids=""
for f in "$REF"/seblas/operations/*.cu "$REF"/seblas/tensor/*.cu "$REF"/seblas/assist/CudaAssert.cu; do
    o="$OUT/obj/$(basename "$f" .cu).o"
    $NVCC $FLAGS -c "$f" -o "$o" &
    pids="$pids $!"
done
$NVCC $FLAGS -c "$HERE/ref/ref_shim.cu" -o "$OUT/obj/ref_shim.o" &
pids="$pids $!"
for p in $pids; do wait "$p"; done
$NVCC -shared -o "$OUT/libseblas_ref.so" "$OUT"/obj/*.o -L/usr/lib/x86_64-linux-gnu -lcudnn -lcurand
rm -rf "$OUT/obj"
echo "$OUT/libseblas_ref.so"
