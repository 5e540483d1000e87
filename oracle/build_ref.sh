#!/usr/bin/env bash
# TEST INFRASTRUCTURE. Compiles the reference's own host sources (unmodified, where they lie in
# the reference checkout, CPU-only stub mode) plus oracle/ref_shim.cpp into
# oracle/_ref/libsca_ref.so. Nothing is copied from the reference; only the built library lands
# in oracle/_ref/ (git-ignored). Usage: oracle/build_ref.sh <reference_root>   (or SCA_REFERENCE_ROOT=<reference_root>)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${SCA_REFERENCE_ROOT:-}}"
OUT="$HERE/_ref"
if [ -z "$REF" ] || [ ! -d "$REF/src" ]; then
    echo "build_ref: no reference checkout given (argument or SCA_REFERENCE_ROOT); skipped"
    exit 0
fi
mkdir -p "$OUT"
SRCS=(
    "$REF/src/api/api_validate.cpp"
    "$REF/src/api/attention_api.cpp"
    "$REF/src/api/status.cpp"
    "$REF/src/runtime/dispatcher.cpp"
    "$REF/src/runtime/backend_lookup.cpp"
    "$REF/src/runtime/capability.cpp"
    "$REF/src/runtime/device_probe_stub.cpp"
    "$REF/src/runtime/scratch_pool.cpp"
    "$REF/src/runtime/workspace.cpp"
    "$REF/src/backends/backends_stub.cpp"
    "$REF/src/backends/naive/naive_backend.cpp"
    "$REF/src/backends/tiled/tiled_backend.cpp"
    "$REF/src/backends/flash/flash_backend.cpp"
    "$REF/src/backends/decode/decode_backend.cpp"
    "$REF/src/backends/paged/paged_backend.cpp"
    "$REF/src/kv_cache/block_manager.cpp"
    "$REF/src/kv_cache/kv_cache.cpp"
    "$REF/src/kv_cache/paged_kv_cache.cpp"
    "$HERE/ref_shim.cpp"
)
g++ -std=c++20 -O2 -fPIC -shared -DSCI_ATTENTION_INFRA_STUB=1 \
    -I "$HERE/ref_shim_include" -I "$REF/stub/include" -I "$REF/include" -I "$REF/src" -I "$REF/tests" \
    "${SRCS[@]}" -o "$OUT/libsca_ref.so"
echo "build_ref: wrote $OUT/libsca_ref.so"
