#!/bin/bash
# Compiles the reference's own sources (cpp/src/*.cu, cpp/src/log.cc), where they lie, into
# oracle/_ref/libcuhnsw_ref.so for the B200 (sm_100).  Needs: the reference checkout, an spdlog
# header tree (one ships inside the flashinfer wheel) and the json11 stand-in in ref_shim/.
# Output stays out of git (oracle/_ref/ is ignored) but travels to the GPU box.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${REFERENCE_ROOT:-$HERE/../../reference}"  # default: a checkout named "reference" beside this repository
SPDLOG="$(python - <<'PY'
import os, importlib.util
spec = importlib.util.find_spec("flashinfer")
print(os.path.join(os.path.dirname(spec.origin), "data", "spdlog", "include") if spec else "")
PY
)"
[ -d "$REF/cpp/src" ] || { echo "no reference checkout at $REF"; exit 0; }
[ -d "$SPDLOG/spdlog" ] || { echo "no spdlog headers found"; exit 0; }
mkdir -p "$HERE/_ref"
OUT="$HERE/_ref/libcuhnsw_ref.so"
if [ -f "$OUT" ] && [ "$OUT" -nt "$HERE/ref_driver.cu" ]; then exit 0; fi
/usr/local/cuda/bin/nvcc -gencode arch=compute_100,code=sm_100 -std=c++17 -O3 -shared -Xcompiler -fPIC,-fopenmp,-w -w \
  -I"$REF/cpp/include" -I"$HERE/ref_shim" -I"$SPDLOG" \
  "$REF/cpp/src/cuhnsw_base.cu" "$REF/cpp/src/cuhnsw_build.cu" "$REF/cpp/src/log.cc" "$HERE/ref_driver.cu" \
  -o "$OUT" -lcudart -lgomp
echo "built $OUT"
