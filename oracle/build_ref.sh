#!/usr/bin/env bash
# Builds oracle/_ref/libgemma4_ref.so from the reference's own sources where they lie (read-only mount),
# for sm_100a, with the flags of the reference's Makefile (NVCCFLAGS, RDC_NVCCFLAGS, FLASH_ATTN_NVCCFLAGS:
# Makefile:6-8,26). TEST INFRASTRUCTURE: a second checker and the source of tests/golden. Outputs go only
# to oracle/_ref/ (git-ignored). The reference's un-vendored CUTLASS submodule is replaced by the CuTe
# headers that ship inside the flashinfer wheel of this image (header-only; used for make_layout only).
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${GEMMA_REF_SRC:-/root/reference/src}"
OUT="$HERE/_ref"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
CUTLASS="${CUTLASS_INCLUDE:-$(python -c 'import flashinfer, os; print(os.path.join(os.path.dirname(flashinfer.__file__), "data/cutlass/include"))')}"
[ -d "$REF" ] || { echo "reference sources not found at $REF" >&2; exit 3; }
[ -d "$CUTLASS/cute" ] || { echo "CuTe headers not found at $CUTLASS" >&2; exit 3; }
mkdir -p "$OUT"
STAMP="$OUT/build.stamp"
KEY="$(cat "$HERE/ref_harness.cu" "$HERE/build_ref.sh" "$REF/gemma4_flash_attention_decode.cu" "$REF/gemma4_flash_attention_prefill.cu" "$REF/gemma4_kv_cache.cu" "$REF/gemma4_rmsnorm.cu" "$REF/gemma4_rope.cu" | sha256sum | cut -d' ' -f1)"
if [ -f "$OUT/libgemma4_ref.so" ] && [ -f "$STAMP" ] && [ "$(cat "$STAMP")" = "$KEY" ]; then exit 0; fi
ARCH="-gencode arch=compute_100a,code=sm_100a"
COMMON="-std=c++17 -O3 $ARCH -rdc=true -Xcompiler -fPIC -I$REF -I$CUTLASS"
FAST="--expt-relaxed-constexpr --expt-extended-lambda --use_fast_math"
$NVCC $COMMON $FAST -c "$HERE/ref_harness.cu" -o "$OUT/ref_harness.o"
# the prompt attention (FA-2 on CuTe) with its two public entry points, src/gemma4_flash_attention.cuh
$NVCC $COMMON $FAST -c "$REF/gemma4_flash_attention_prefill.cu" -o "$OUT/gemma4_flash_attention_prefill.o"
$NVCC $COMMON -c "$REF/gemma4_rmsnorm.cu" -o "$OUT/gemma4_rmsnorm.o"
$NVCC $COMMON -c "$REF/gemma4_rope.cu" -o "$OUT/gemma4_rope.o"
$NVCC $COMMON -c "$REF/gemma4_kv_cache.cu" -o "$OUT/gemma4_kv_cache.o"
$NVCC $ARCH -Xcompiler -fPIC -shared "$OUT/ref_harness.o" "$OUT/gemma4_flash_attention_prefill.o" "$OUT/gemma4_rmsnorm.o" "$OUT/gemma4_rope.o" "$OUT/gemma4_kv_cache.o" -o "$OUT/libgemma4_ref.so"
echo "$KEY" > "$STAMP"
echo "built $OUT/libgemma4_ref.so"
