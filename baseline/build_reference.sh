#!/bin/bash
# Builds the unmodified reference single-GPU trainer for sm_100, one binary per hidden size, under baseline/_ref.
# Usage: baseline/build_reference.sh [/path/to/reference/FINAL_CLEAN_CODE_]
#        (default: $CME213_REFERENCE_DIR/FINAL_CLEAN_CODE_, else the checkout next to this repository)
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
SRC=${1:-${CME213_REFERENCE_DIR:-$HERE/../../reference}/FINAL_CLEAN_CODE_}
DST="$(cd "$(dirname "$0")" && pwd)/_ref"
mkdir -p "$DST"
cp -r "$SRC/Makefile" "$SRC/include" "$SRC/src" "$SRC/inp.txt" "$DST/"
cd "$DST"
for H in 128 256 512; do
  make -j8 CUDA_ARCH=-arch=sm_100 CUDA_LIB_DIR=/usr/local/cuda/lib64 CUBLAS_LIB_DIR=/usr/local/cuda/lib64 \
       BUILD_DIR=build_h$H EXTRA_NVCC_FLAGS="-DHIDDEN_DIM=$H" > build_h$H.log 2>&1
  ls -la build_h$H/train
done
