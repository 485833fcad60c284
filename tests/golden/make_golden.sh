#!/bin/bash
# Builds make_golden.cpp against a checkout of celsowm/celeg (first argument, required) with g++ on the
# CPU and writes golden.json beside this script. Only the reference's plain float32 kernels are linked:
# elementwise, rope, convolution, sampler, the paged attention with its page pool and pattern policy, ISA
# detection, the thread pool and the topology probe they need.
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:?usage: make_golden.sh /path/to/celeg}"
build="$(mktemp -d)"
srcs=(src/backend/cpu/kernels/elementwise.cpp src/backend/cpu/kernels/rope.cpp
      src/backend/cpu/kernels/convolution.cpp src/backend/cpu/sampler.cpp
      src/backend/cpu/attention/paged_attention.cpp src/backend/cpu/memory/paged_kv.cpp
      src/backend/cpu/memory/attention_policy.cpp src/model/weights/quantization.cpp
      src/backend/cpu/runtime/numa.cpp
      src/backend/cpu/runtime/isa.cpp src/backend/cpu/runtime/thread_pool.cpp
      src/backend/cpu/runtime/topology.cpp)
args=()
for s in "${srcs[@]}"; do args+=("$ref/$s"); done
g++ -std=c++20 -O1 -I"$ref/include" -I"$ref/src/backend/cpu" -I"$ref/src/backend/cpu/kernels" \
    "$here/make_golden.cpp" "${args[@]}" -lpthread -o "$build/make_golden"
"$build/make_golden" > "$here/golden.json"
echo "wrote $here/golden.json"
