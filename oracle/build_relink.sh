#!/bin/sh
# Relinks the REFERENCE's own operand layer against this library: compiles, from where they lie in the reference
# tree, every seann source (operands, optimizers, containers) and the reference's .crseq codec
# (seio/modelcache/*.cu), with crusaderbackend_b200/compat/ standing where the reference's seblas/ and seio headers
# stood, and links them with tests/cpp/relink_driver.cu and libcrusader_b200.so into oracle/_ref/relink_driver.
#
# The reference's sources include their neighbours by relative path ("../../seblas/operations/cuOperations.cuh"), and a
# quoted include is looked up beside the including file first, so putting compat/ on the include path would not be
# enough. The script therefore builds a shadow tree under oracle/_ref/relink/ (git-ignored) made of real directories
# whose FILES are symbolic links to the reference's sources — nothing is copied — and whose seblas/, seio/logging,
# seio/data and seann/operands/cudnn entries point at compat/. The only reference files left out are
# seann/operands/cudnn/cuConv2D.{cu,cuh} (the cuDNN-backed operand this library replaces under the same name).
# Usage: oracle/build_relink.sh [reference_root]   (default: where the reference tree is mounted, see REF below)
set -e
REF="${1:-/root/reference}"
HERE="$(cd "$(dirname "$0")" && pwd)"
ROOT="$(dirname "$HERE")"
COMPAT="$ROOT/crusaderbackend_b200/compat"
OUT="$HERE/_ref"
SH="$OUT/relink"
if [ ! -d "$REF/seann" ]; then
    echo "build_relink: $REF/seann not found (the reference tree is not mounted); keeping any prebuilt binary" >&2
    exit 0
fi
rm -rf "$SH"
mkdir -p "$SH/obj" "$SH/seio"
# real directories, file-level links
(cd "$REF" && find seann seio/modelcache -type d) | while read -r d; do mkdir -p "$SH/$d"; done
(cd "$REF" && find seann seio/modelcache -type f \( -name '*.cu' -o -name '*.cuh' \)) | while read -r f; do
    case "$f" in seann/operands/cudnn/*) continue ;; esac
    ln -s "$REF/$f" "$SH/$f"
done
ln -s "$COMPAT/seblas" "$SH/seblas"
ln -s "$COMPAT/seio/logging" "$SH/seio/logging"
ln -s "$COMPAT/seio/data" "$SH/seio/data"
ln -s "$COMPAT/seann/operands/cudnn/cuConv2D.cuh" "$SH/seann/operands/cudnn/cuConv2D.cuh"
NVCC="${NVCC:-nvcc}"
FLAGS="-std=c++17 -O2 -gencode arch=compute_100a,code=sm_100a -x cu -w -I$SH"
pids=""
for f in $(cd "$SH" && find seann seio/modelcache -name '*.cu'); do
    o="$SH/obj/$(echo "$f" | tr '/' '_' | sed 's/\.cu$/.o/')"
    $NVCC $FLAGS -c "$SH/$f" -o "$o" &
    pids="$pids $!"
done
$NVCC $FLAGS -c "$ROOT/tests/cpp/relink_driver.cu" -o "$SH/obj/relink_driver.o" &
pids="$pids $!"
for p in $pids; do wait "$p"; done
$NVCC -o "$OUT/relink_driver" "$SH"/obj/*.o -L"$ROOT/crusaderbackend_b200/lib" -lcrusader_b200 \
    -Xlinker -rpath -Xlinker '$ORIGIN/../../crusaderbackend_b200/lib'
rm -rf "$SH"
echo "$OUT/relink_driver"
