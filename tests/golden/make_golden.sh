#!/bin/sh
# Compiles the reference's own scheduler, block pool, host sampler, configuration parser and
# safetensors reader
# (unmodified sources of
# a divedb/InferX checkout given as $1) on the CPU, against the small stand-in for abseil in
# absl_stub/ (and for the two mimalloc calls of its host allocator), links them with the four drivers of this folder and writes what they print to
# scheduler_golden.jsonl, sampling_golden.jsonl, config_golden.jsonl and checkpoint_golden.jsonl
# (the last over a model folder that this repository's write_random_model writes first, so
# python and torch are needed for that one).  tests/test_scheduler_golden.py reads
# those files; it needs neither the checkout nor a compiler.
#
#   sh tests/golden/make_golden.sh /path/to/InferX
set -e
REF=${1:?usage: make_golden.sh /path/to/InferX}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$(mktemp -d)
INC="-I$HERE/absl_stub -I$REF/include -I$REF/src/core"
n=0
for f in src/scheduler/scheduler.cc src/scheduler/prefix_cache.cc src/core/kv_cache.cc \
         src/core/device_buffer.cc src/core/tensor_view.cc src/core/shape.cc \
         src/core/device_runtime.cc src/backends/cpu/device_runtime.cc \
         src/core/accelerator_runtime_stub.cc src/engine/host_sampling.cc \
         src/model/config.cc src/support/json.cc src/model/safetensors.cc \
         src/core/tensor.cc src/core/storage.cc src/core/allocator.cc; do
  n=$((n + 1))
  g++ -std=c++20 -O1 $INC -c "$REF/$f" -o "$OUT/ref_$n.o"
done
g++ -std=c++20 -O1 $INC -c "$HERE/scheduler_golden.cc" -o "$OUT/scheduler_golden.o"
g++ -std=c++20 -O1 $INC -c "$HERE/sampling_golden.cc" -o "$OUT/sampling_golden.o"
g++ -std=c++20 -O1 $INC -c "$HERE/config_golden.cc" -o "$OUT/config_golden.o"
g++ -std=c++20 -O1 $INC -c "$HERE/checkpoint_golden.cc" -o "$OUT/checkpoint_golden.o"
g++ "$OUT"/ref_*.o "$OUT/scheduler_golden.o" -o "$OUT/scheduler_golden"
g++ "$OUT"/ref_*.o "$OUT/sampling_golden.o" -o "$OUT/sampling_golden"
g++ "$OUT"/ref_*.o "$OUT/config_golden.o" -o "$OUT/config_golden"
g++ "$OUT"/ref_*.o "$OUT/checkpoint_golden.o" -o "$OUT/checkpoint_golden"
"$OUT/scheduler_golden" > "$HERE/scheduler_golden.jsonl"
"$OUT/sampling_golden" > "$HERE/sampling_golden.jsonl"
"$OUT/config_golden" "$HERE"/config_cases/*.json > "$HERE/config_golden.jsonl"
(cd "$HERE/../.." && python -c "
import json, sys
from inferx_b200.weights.random_model import write_random_model
write_random_model(json.load(open('tests/golden/config_cases/tiny_b.json')), sys.argv[1], seed=7, dtype='bfloat16')
" "$OUT/model")
"$OUT/checkpoint_golden" "$OUT/model" > "$HERE/checkpoint_golden.jsonl"
wc -l "$HERE/scheduler_golden.jsonl" "$HERE/sampling_golden.jsonl" "$HERE/config_golden.jsonl" "$HERE/checkpoint_golden.jsonl"
rm -r "$OUT"
