#!/usr/bin/env bash
# Builds the UNMODIFIED reference torch extension (rptc_kernels/csrc/rptc_kernels/{wrapper.cpp,
# inference.cu,inference_t.cu}, flags of rptc_kernels/setup.py:12-17 plus an sm_100a -gencode)
# straight from the read-only reference checkout into oracle/_ref/.  Nothing is copied: the
# sources are compiled where they lie.  The resulting module is test infrastructure only: the GPU
# parity tests import it as `rptc_kernels_reference` to pin the CPU oracle's "refkernel" mode
# against what the reference's own kernels really compute.
#
#   usage: oracle/build_ref.sh [reference_root]      (default: $RPTC_REFERENCE_ROOT, else ../reference beside this repository)
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${1:-${RPTC_REFERENCE_ROOT:-$(dirname "$(dirname "$HERE")")/reference}}"
SRC="$REF/rptc_kernels/csrc/rptc_kernels"
OUT="$HERE/_ref"
[ -d "$SRC" ] || { echo "reference sources not found under $SRC" >&2; exit 3; }
mkdir -p "$OUT/obj"
PY="${PYTHON:-python}"
TORCH_DIR="$($PY -c 'import torch,os;print(os.path.dirname(torch.__file__))' 2>/dev/null)"
PYINC="$($PY -c 'import sysconfig;print(sysconfig.get_paths()["include"])')"
EXT="$($PY -c 'import sysconfig;print(sysconfig.get_config_var("EXT_SUFFIX"))')"
NAME=rptc_kernels_reference
INC=(-I"$TORCH_DIR/include" -I"$TORCH_DIR/include/torch/csrc/api/include" -I"$PYINC")
DEF=(-DTORCH_EXTENSION_NAME=$NAME -DTORCH_API_INCLUDE_EXTENSION_H -D_GLIBCXX_USE_CXX11_ABI=1)
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
for f in inference inference_t; do
  "$NVCC" -c "$SRC/$f.cu" -o "$OUT/obj/$f.o" "${INC[@]}" "${DEF[@]}" \
      -gencode arch=compute_100a,code=sm_100a -O3 --use_fast_math -lineinfo -std=c++17 \
      -Xcompiler -fPIC --expt-relaxed-constexpr &
done
g++ -c "$SRC/wrapper.cpp" -o "$OUT/obj/wrapper.o" "${INC[@]}" "${DEF[@]}" -O3 -std=c++17 -fPIC &
wait
g++ -shared "$OUT/obj/wrapper.o" "$OUT/obj/inference.o" "$OUT/obj/inference_t.o" -o "$OUT/$NAME$EXT" \
    -L"$TORCH_DIR/lib" -L/usr/local/cuda/lib64 -lc10 -lc10_cuda -ltorch_cpu -ltorch_cuda -ltorch -ltorch_python -lcudart \
    -Wl,-rpath,"$TORCH_DIR/lib"
echo "built $OUT/$NAME$EXT"
