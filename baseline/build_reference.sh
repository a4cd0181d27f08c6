#!/bin/bash
# Compiles the reference project's own kernel (its csrc/kernels/gemm.cu and bindings.cpp, unmodified, read where
# they lie) for sm_100 into baseline/_ref/gemm_int8_CUDA.so, against the CUTLASS headers that ship inside the
# flashinfer Python package and the installed libtorch.  The result is the reference's Sm80 mma.sync template
# recompiled for Blackwell: the same-box comparator of the dense GEMM and the pin of the CPU oracle.
# Nothing is copied into the repository; baseline/_ref/ is ignored by git.
#
# usage: baseline/build_reference.sh [path of the reference checkout]   (takes about three minutes)
# Without an argument: $GEMM_INT8_REFERENCE, else a checkout named "reference" beside this repository.
set -euo pipefail
HERE=$(cd "$(dirname "$0")" && pwd)
REF=${1:-${GEMM_INT8_REFERENCE:-$HERE/../../reference}}
OUT=$HERE/_ref
SRC=$REF/csrc/kernels
[ -f "$SRC/gemm.cu" ] || { echo "reference sources not found under $REF" >&2; exit 2; }
PY=${PYTHON:-python}
read -r TORCH_DIR CUTLASS_DIR PY_INC ABI <<<"$($PY - <<'PYEOF'
import os, sysconfig, torch, importlib.util
spec = importlib.util.find_spec("flashinfer")
cut = os.path.join(os.path.dirname(spec.origin), "data", "cutlass")
print(os.path.dirname(torch.__file__), cut, sysconfig.get_paths()["include"], int(torch._C._GLIBCXX_USE_CXX11_ABI))
PYEOF
)"
[ -d "$CUTLASS_DIR/include/cutlass" ] || { echo "no CUTLASS headers under $CUTLASS_DIR" >&2; exit 2; }
mkdir -p "$OUT"
INC=(-I"$SRC/include" -I"$CUTLASS_DIR/include" -I"$CUTLASS_DIR/tools/util/include"
     -I"$TORCH_DIR/include" -I"$TORCH_DIR/include/torch/csrc/api/include" -I"$PY_INC" -I/usr/local/cuda/include)
DEF=(-D_GLIBCXX_USE_CXX11_ABI=$ABI -DTORCH_EXTENSION_NAME=gemm_int8_CUDA)
nvcc -std=c++17 -O2 --expt-relaxed-constexpr --use_fast_math -Xcompiler -fPIC \
     -gencode arch=compute_100,code=sm_100 "${INC[@]}" "${DEF[@]}" -c "$SRC/gemm.cu" -o "$OUT/gemm.o" &
g++ -std=c++17 -O2 -fPIC "${INC[@]}" "${DEF[@]}" -c "$SRC/bindings.cpp" -o "$OUT/bindings.o" &
wait
g++ -shared -o "$OUT/gemm_int8_CUDA.so" "$OUT/gemm.o" "$OUT/bindings.o" \
    -L"$TORCH_DIR/lib" -ltorch -ltorch_cpu -ltorch_cuda -lc10 -lc10_cuda -L/usr/local/cuda/lib64 -lcudart \
    -Wl,-rpath,"$TORCH_DIR/lib"
rm -f "$OUT/gemm.o" "$OUT/bindings.o"
echo "built $OUT/gemm_int8_CUDA.so"
