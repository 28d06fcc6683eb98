#!/usr/bin/env bash
# Builds the NeuZephyr reference itself (its own sources, left where they lie) for sm_100
# plus the A/B harness, into oracle/_ref/. Test infrastructure only; nothing here is
# part of the product. Usage: bash build_ref.sh /path/to/NeuZephyr
#
# The reference's CMake build targets "native" and MSVC; with gcc 13 + nvcc 12.9 it needs
# a handful of force-included standard headers and two one-token fixes for an ambiguous
# brace construction (src/Dimension.cu:129, src/Tensor.cu:89). Those two edits are applied
# to a scratch copy under a temporary directory; only binaries are written to _ref/.
set -euo pipefail
REF="${1:-${NEUZEPHYR_SRC:-}}"
[ -n "$REF" ] || { echo "usage: build_ref.sh /path/to/NeuZephyr (or set NEUZEPHYR_SRC)" >&2; exit 3; }
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
[ -d "$REF/src" ] || { echo "reference sources not found at $REF" >&2; exit 3; }
mkdir -p "$OUT"
TMP="$(mktemp -d /tmp/nzref.XXXXXX)"
trap 'rm -rf "$TMP"' EXIT
cp "$REF"/src/*.cu "$TMP"/
sed -i 's/Dimension result({0, 0, 0, 0})/Dimension result(0, 0, 0, 0)/' "$TMP/Dimension.cu"
sed -i 's/_shape({0, 0, 0, 0})/_shape(0, 0, 0, 0)/' "$TMP/Tensor.cu"
INC=(-include condition_variable -include memory -include algorithm -include string -include mutex
     -include queue -include unordered_map -include unordered_set -include chrono -include iomanip
     -include memory_resource -include stdexcept -include numeric)
FLAGS=(-std=c++17 -arch=sm_100 -O3 -w -Xcompiler -fPIC -DNEUZEPHYR_EXPORTS -I"$REF/include" "${INC[@]}")
pids=()
for f in "$TMP"/*.cu; do
  "$NVCC" "${FLAGS[@]}" -dc "$f" -o "${f%.cu}.o" &
  pids+=($!)
done
for p in "${pids[@]}"; do wait "$p"; done
"$NVCC" -arch=sm_100 -shared "$TMP"/*.o -lcurand -o "$OUT/libNeuZephyr.so"
"$NVCC" "${FLAGS[@]}" "$HERE/ref_harness.cu" -L"$OUT" -lNeuZephyr -lcurand -Xlinker -rpath -Xlinker '$ORIGIN' \
  -o "$OUT/ref_harness"
echo "built $OUT/libNeuZephyr.so and $OUT/ref_harness"
