#!/bin/bash
# Whole-model anchor: celsowm/celeg's CPU model on the tiny-A random-weights folder.
#   make_golden_model.sh /path/to/celeg /path/to/folder/with/libceleg.so
# The library is the one baseline/build_reference.py builds (celeg's own sources, unmodified). The model
# folder is written here by this repository's seeded random-weights writer (tiny A, seed 0, bfloat16), the
# same folder tests/test_golden_reference.py writes again when it compares. Writes golden_model.json beside
# this script.
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:?usage: make_golden_model.sh /path/to/celeg /path/to/libceleg/folder}"
lib="${2:?usage: make_golden_model.sh /path/to/celeg /path/to/libceleg/folder}"
build="$(mktemp -d)"
(cd "$here/.." && python - "$build" <<'PY'
import sys, pathlib
sys.path.insert(0, ".")
sys.path.insert(0, "..")
import tiny_models
print(tiny_models.write_tiny(pathlib.Path(sys.argv[1]), "A"))
PY
)
g++ -std=c++20 -O1 -I"$ref/include" "$here/make_golden_model.cpp" -L"$lib" -Wl,-rpath,"$lib" -lceleg -lpthread \
    -o "$build/make_golden_model"
"$build/make_golden_model" "$build/tiny_A" 5 17 3 250 9 41 77 300 12 > "$here/golden_model.json"
echo "wrote $here/golden_model.json"
