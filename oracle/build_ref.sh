#!/bin/sh
# Builds oracle/_ref/libref_oracle.so from the REFERENCE's own C++ CPU ops.
# Test infrastructure only.  Reads the reference checkout (default
# /root/reference, override with REFERENCE_ROOT), writes only under
# oracle/_ref/ (git-ignored; no reference source is ever committed).
#
# The reference targets macOS; four mechanical transforms make its CPU path
# compile with g++ on Linux (each applied to a scratch copy in _ref/src):
#  1. Accelerate / GCD headers come from oracle/shim (plain-loop stand-ins).
#  2. Weight constructors say DType::BF16 while every CPU branch reads the
#     buffers as float; DType::BF16 -> DType::FP32 restores the fp32 CPU engine.
#     Tensor.cpp is compiled unmodified.
#  3. The two dispatch_apply(^block) loops in Attention.cpp become
#     shim_parallel_for(lambda) (g++ has no blocks extension).
#  4. Alias fix: Tensor copies are shallow, so swiglu() clobbers its gate
#     argument and h_cache_ aliases every cached hidden state; two clone()
#     calls give the mathematically intended behaviour.  ALIAS_FIX=0 builds the
#     as-is variant (_ref/libref_oracle_asis.so) used only to report the delta.
#  5. Checkpoint::save fills a local SavedTensor whose `data` points into its own `owned_data` vector, then
#     push_back()s a COPY of it: the copy's `data` still points into the local, which is destroyed at the end of
#     the block, so every transposed tensor is written from freed memory (cpp/src/Checkpoint.cpp:736-742, 706-713).
#     The fixed variant makes the writer prefer the element's own `owned_data`; the file layout is unchanged.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${REFERENCE_ROOT:-$HERE/../../reference}"   # default: a checkout named "reference" beside this repository
ALIAS_FIX="${ALIAS_FIX:-1}"
CXX_BIN="${ORC_CXX:-g++}"
[ -d "$REF/cpp/src" ] || { echo "reference checkout not found at $REF: set REFERENCE_ROOT to the directory that holds its cpp/src" >&2; exit 3; }
OUT="$HERE/_ref"
SRC="$OUT/src_fix$ALIAS_FIX"
mkdir -p "$SRC"
for f in RMSNorm Activations Positional Loss Transformer Optimizer Attention Checkpoint Trainer DataIngestion; do
  sed 's/DType::BF16/DType::FP32/g' "$REF/cpp/src/$f.cpp" > "$SRC/$f.cpp"
done
cp "$REF/cpp/src/Tensor.cpp" "$SRC/Tensor.cpp"
python3 - "$SRC/Attention.cpp" <<'PY'
import re, sys
p = sys.argv[1]
s = open(p).read()
pat = re.compile(r"dispatch_apply\(\s*batch \* n_h,\s*dispatch_get_global_queue\(DISPATCH_QUEUE_PRIORITY_HIGH, 0\),\s*\^\(size_t bh\) \{")
s, n = pat.subn("shim_parallel_for(batch * n_h, [&](size_t bh) {", s)
assert n == 2, f"expected 2 dispatch_apply sites, found {n}"
open(p, "w").write(s)
PY
if [ "$ALIAS_FIX" = "1" ]; then
  sed -i 's/Tensor gated = gate;/Tensor gated = gate.clone();/' "$SRC/Activations.cpp"
  sed -i 's/h_cache_.push_back(h);/h_cache_.push_back(h.clone());/g' "$SRC/Transformer.cpp"
  grep -q 'gate.clone()' "$SRC/Activations.cpp"
  [ "$(grep -c 'push_back(h.clone())' "$SRC/Transformer.cpp")" = "2" ]
  sed -i 's/reinterpret_cast<const char \*>(tensors\[i\].data),/reinterpret_cast<const char *>(tensors[i].owned_data.empty() ? tensors[i].data : tensors[i].owned_data.data()),/' "$SRC/Checkpoint.cpp"
  [ "$(grep -c 'owned_data.empty() ? tensors' "$SRC/Checkpoint.cpp")" = "1" ]
  LIB="$OUT/libref_oracle.so"
else
  LIB="$OUT/libref_oracle_asis.so"
fi
$CXX_BIN -std=c++20 -O2 -fopenmp -fPIC -shared -fvisibility=hidden -ffp-contract=off \
  -include chrono -include string -include numeric -include cstring -include thread \
  -I"$HERE/shim" -I"$REF/cpp/include" \
  "$SRC"/*.cpp "$HERE/shim/bridge_cpu_stub.cpp" "$HERE/ref_driver.cpp" -o "$LIB" -lpthread
echo "built $LIB"
# Drop-in check (alias-fixed variant only): the same reference sources and driver, linked against the
# B200 backend's `namespace metal_bridge` adaptor instead of the CPU stub.  With GPU_ENABLED=1 every op of
# the reference engine then runs on the CUDA kernels through host pointers (tests/test_gpu_dropin.py).
PKGDIR="$HERE/../large-language-model_b200"
if [ "$ALIAS_FIX" = "1" ] && [ -f "$PKGDIR/libb200bridge.so" ]; then
  $CXX_BIN -std=c++20 -O2 -fopenmp -fPIC -shared -fvisibility=hidden -ffp-contract=off \
    -include chrono -include string -include numeric -include cstring -include thread \
    -I"$HERE/shim" -I"$REF/cpp/include" -I"$HERE/../include" \
    "$SRC"/*.cpp "$PKGDIR/adaptor/metal_bridge_b200.cpp" "$HERE/ref_driver.cpp" \
    -o "$OUT/libref_on_b200.so" -L"$PKGDIR" -lb200bridge -Wl,-rpath,'$ORIGIN/../../large-language-model_b200' -lpthread
  echo "built $OUT/libref_on_b200.so"
  # the same with bf16 device mirrors (what the reference's Metal shaders read): the reference engine then runs on the
  # tensor-core kernels; parity gate 2e-2
  $CXX_BIN -std=c++20 -O2 -fopenmp -fPIC -shared -fvisibility=hidden -ffp-contract=off -DB200_ADAPTOR_BF16 \
    -include chrono -include string -include numeric -include cstring -include thread \
    -I"$HERE/shim" -I"$REF/cpp/include" -I"$HERE/../include" \
    "$SRC"/*.cpp "$PKGDIR/adaptor/metal_bridge_b200.cpp" "$HERE/ref_driver.cpp" \
    -o "$OUT/libref_on_b200_bf16.so" -L"$PKGDIR" -lb200bridge -Wl,-rpath,'$ORIGIN/../../large-language-model_b200' -lpthread
  echo "built $OUT/libref_on_b200_bf16.so"
fi
