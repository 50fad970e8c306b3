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
ARCH="-gencode arch=compute_100a,code=sm_100a"
if ! { [ -f "$OUT/libgemma4_ref.so" ] && [ -f "$STAMP" ] && [ "$(cat "$STAMP")" = "$KEY" ]; }; then
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
fi

# The drop-in proof: the reference's own test programs, unchanged, compiled against the library's stand-in headers
# (include/compat ahead of the reference's src/) and linked to libgemma4_b200kv.so -- no reference object in the
# link -- plus tests/cpp/megakernel_layer.cu, which includes the reference's real gemma4_megakernel.cuh. They run
# on the GPU (tests/test_gpu_reference_boundary.py). Needs the library built first (gemma.c_b200/build.py).
REPO="$(cd "$HERE/.." && pwd)"
LIBDIR="$REPO/gemma.c_b200/_build"
TESTS="$(cd "$REF/../tests" 2>/dev/null && pwd || true)"
if [ -f "$LIBDIR/libgemma4_b200kv.so" ] && [ -n "$TESTS" ] && [ -f "$TESTS/test_kv_cache.cu" ]; then
  TKEY="$(cat "$HERE/build_ref.sh" "$REPO"/include/*.h* "$REPO"/include/compat/*.cuh "$REPO/tests/cpp/megakernel_layer.cu" \
          "$TESTS/test_kv_cache.cu" "$TESTS/test_runtime_state.cu" "$TESTS/test_flash_attention.cu" \
          "$REF/gemma4_megakernel.cuh" "$REF/gemma4.h" | sha256sum | cut -d' ' -f1)"
  TSTAMP="$OUT/boundary.stamp"
  if ! { [ -f "$OUT/ref_test_kv_cache" ] && [ -f "$OUT/megakernel_layer" ] && [ -f "$TSTAMP" ] && [ "$(cat "$TSTAMP")" = "$TKEY" ]; }; then
    LINK="-L$LIBDIR -lgemma4_b200kv -Xlinker -rpath -Xlinker \$ORIGIN/../../gemma.c_b200/_build"
    for t in test_kv_cache test_runtime_state test_flash_attention; do
      $NVCC -std=c++17 -O2 $ARCH -I"$REPO/include/compat" -I"$REPO/include" -I"$REF" "$TESTS/$t.cu" $LINK -o "$OUT/ref_$t"
    done
    $NVCC -std=c++17 -O2 $ARCH -I"$REF" -I"$REPO/include" "$REPO/tests/cpp/megakernel_layer.cu" $LINK -o "$OUT/megakernel_layer"
    echo "$TKEY" > "$TSTAMP"
    echo "built $OUT/ref_test_{kv_cache,runtime_state,flash_attention} and $OUT/megakernel_layer"
  fi
fi
