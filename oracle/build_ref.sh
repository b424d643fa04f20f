#!/usr/bin/env bash
# Compile the UNMODIFIED reference sources (read where they lie, never copied) for sm_100
# into oracle/_ref/libgs_ref.so.  The reference is CUDA-only, so the library can be loaded
# anywhere torch is present but its ops only run on a GPU box.  Used as (a) the bit-exact
# checker for deterministic ops when fixtures are generated and (b) the reference arm of
# bench.py.  Usage: oracle/build_ref.sh [REFERENCE_ROOT] [JOBS]
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-/root/reference}"
JOBS="${2:-8}"
OUT="$HERE/_ref"
OBJ="$OUT/obj"
mkdir -p "$OBJ"
if [ ! -d "$REF/src" ]; then echo "reference sources not found at $REF" >&2; exit 3; fi
PY=python
TORCH=$($PY -c 'import torch,os;print(os.path.dirname(torch.__file__))')
PYINC=$($PY -c 'import sysconfig;print(sysconfig.get_paths()["include"])')
FLAGS=(-std=c++17 --extended-lambda --expt-relaxed-constexpr
  -gencode arch=compute_100,code=sm_100 -D_GLIBCXX_USE_CXX11_ABI=1 -Xcompiler -fPIC -O3 -w
  -I "$HERE/ref_shim" -I "$REF/src" -I "$REF/src/cuda"
  -I "$TORCH/include" -I "$TORCH/include/torch/csrc/api/include" -I "$PYINC")
compile_one() {
  src="$1"; name="$(echo "${src#$REF/}" | tr '/' '_')"; obj="$OBJ/${name%.*}.o"
  if [ -f "$obj" ] && [ "$obj" -nt "$src" ]; then return 0; fi
  extra=()
  case "$src" in *.cc) extra=(-x cu);; esac
  nvcc "${FLAGS[@]}" "${extra[@]}" -c "$src" -o "$obj"
}
export -f compile_one; export REF OBJ HERE
pids=()
running=0
for src in "$REF"/src/*.cc "$REF"/src/cuda/*.cu "$REF"/src/cuda/fusion/*.cu; do
  ( compile_one "$src" && echo "ok $src" || { echo "FAILED $src"; exit 1; } ) &
  running=$((running+1))
  if [ "$running" -ge "$JOBS" ]; then wait -n; running=$((running-1)); fi
done
wait
n_obj=$(ls "$OBJ"/*.o | wc -l)
echo "objects: $n_obj"
nvcc -shared -o "$OUT/libgs_ref.so" "$OBJ"/*.o -L"$TORCH/lib" -ltorch -ltorch_cpu -ltorch_cuda -lc10 -lc10_cuda
echo "built $OUT/libgs_ref.so"
