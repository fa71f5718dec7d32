#!/bin/sh
# Builds the reference's own CUDA signature kernels (unmodified sources, compiled where
# they lie) into oracle/_ref/libcusig_ref.so for same-GPU parity checks and timing.
# Only two translation units are needed for signature_cuda_* / sig_backprop_cuda_*:
# siglib/cusig/cu_signature.cu and siglib/cusig/cu_path_transforms.cu (no Highway, oneTBB
# or preparation library).  The reference's build system is not used.
#   usage: oracle/build_ref_cuda.sh /path/to/reference     (takes 15-40 min of compiler time)
set -e
REF="${1:?usage: build_ref_cuda.sh /path/to/reference}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT"
nvcc -std=c++20 -O2 -gencode arch=compute_100a,code=sm_100a -DCUSIG_EXPORTS -DNDEBUG \
     -I "$REF/siglib/cusig" -I "$REF/siglib/shared" -I "$REF/siglib" \
     --split-compile 3 -shared -Xcompiler -fPIC \
     "$REF/siglib/cusig/cu_signature.cu" "$REF/siglib/cusig/cu_path_transforms.cu" \
     -o "$OUT/libcusig_ref.so"
echo "built $OUT/libcusig_ref.so"
