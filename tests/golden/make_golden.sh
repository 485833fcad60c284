#!/bin/bash
# Builds make_golden.cpp against a checkout of celsowm/celeg (first argument, default /root/reference)
# with g++ on the CPU and writes golden.json beside this script. Only the reference's plain float32
# kernels are linked: elementwise, rope, convolution, sampler, ISA detection, the thread pool and the topology probe it needs.
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:-/root/reference}"
build="$(mktemp -d)"
srcs=(src/backend/cpu/kernels/elementwise.cpp src/backend/cpu/kernels/rope.cpp
      src/backend/cpu/kernels/convolution.cpp src/backend/cpu/sampler.cpp
      src/backend/cpu/runtime/isa.cpp src/backend/cpu/runtime/thread_pool.cpp
      src/backend/cpu/runtime/topology.cpp)
args=()
for s in "${srcs[@]}"; do args+=("$ref/$s"); done
g++ -std=c++20 -O1 -I"$ref/include" -I"$ref/src/backend/cpu" -I"$ref/src/backend/cpu/kernels" \
    "$here/make_golden.cpp" "${args[@]}" -lpthread -o "$build/make_golden"
"$build/make_golden" > "$here/golden.json"
echo "wrote $here/golden.json"
