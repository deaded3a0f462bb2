#!/bin/bash
# TEST INFRASTRUCTURE.  Compiles the unmodified reference (main.cu + its generated
# kernels, read in place from $REF) behind oracle/ref_harness.cu for sm_100a.
# Outputs go only to oracle/_ref/ (git-ignored): libturbofft_ref.so and a copy of
# the reference's A100 parameter tables, which its launch protocol reads at run time.
# Needs the reference tree ($TURBOFFT_REFERENCE, else a checkout named "reference" beside this
# repository); on a machine without it the prebuilt files are used as is.
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${TURBOFFT_REFERENCE:-$HERE/../../reference}"
OUT="$HERE/_ref"
if [ ! -f "$REF/main.cu" ]; then
    echo "[build_ref] reference tree not found at $REF; keeping prebuilt $OUT" >&2
    exit 0
fi
mkdir -p "$OUT/param/A100"
cp "$REF/include/param/A100/param_float2.csv" "$REF/include/param/A100/param_double2.csv" "$OUT/param/A100/"
if [ "$OUT/libturbofft_ref.so" -nt "$HERE/ref_harness.cu" ]; then
    echo "[build_ref] up to date"
    exit 0
fi
nvcc -std=c++17 -O3 -w -DARCH_SM=80 -gencode arch=compute_100a,code=sm_100a \
    -I"$HERE/ref_shim" -I"$REF" -I"$REF/include" \
    -Xcompiler -fPIC -shared -o "$OUT/libturbofft_ref.so" "$HERE/ref_harness.cu" -lcufft -lcublas
echo "[build_ref] built $OUT/libturbofft_ref.so"
