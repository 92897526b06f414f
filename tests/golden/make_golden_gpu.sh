#!/bin/sh
# Builds ops_golden.cu against the reference's own CUDA kernels (unmodified
# src/backends/cuda/ops/layers.cu and moe.cu of a divedb/InferX checkout given as $1,
# compiled for sm_100a with the stand-in for abseil in absl_stub/) into the program $2.
# Run that program on a machine with a GPU with an output folder as its argument; it writes
# ops_golden.bin and ops_golden.jsonl, which are committed in this folder.
# tests/test_ops_golden.py reads those two files; it needs neither the checkout nor a GPU.
# A third argument names another driver in this folder to build instead
# (reference_kernel_times.cu: the same kernels timed at the bench's sizes).
#
#   sh tests/golden/make_golden_gpu.sh /path/to/InferX /tmp/ops_golden && /tmp/ops_golden tests/golden
#   sh tests/golden/make_golden_gpu.sh /path/to/InferX /tmp/ref_times reference_kernel_times.cu && /tmp/ref_times
set -e
REF=${1:?usage: make_golden_gpu.sh /path/to/InferX OUTPUT_PROGRAM}
PROG=${2:?usage: make_golden_gpu.sh /path/to/InferX OUTPUT_PROGRAM}
DRIVER=${3:-ops_golden.cu}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$(mktemp -d)
INC="-I$HERE/absl_stub -I$REF/include -I$REF/src/core"
ARCH="-gencode arch=compute_100a,code=sm_100a"
n=0
for f in src/backends/cuda/ops/layers.cu src/backends/cuda/ops/moe.cu \
         src/backends/cuda/cuda_utils.cc src/core/tensor_view.cc src/core/shape.cc; do
  n=$((n + 1))
  nvcc -std=c++20 -O2 -DINFERX_WITH_CUDA -x cu $ARCH $INC -c "$REF/$f" -o "$OUT/ref_$n.o"
done
nvcc -std=c++20 -O2 -DINFERX_WITH_CUDA $ARCH $INC -c "$HERE/$DRIVER" -o "$OUT/driver.o"
nvcc $ARCH "$OUT"/ref_*.o "$OUT/driver.o" -o "$PROG"
rm -r "$OUT"
echo "built $PROG"
