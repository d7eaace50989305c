#!/usr/bin/env bash
# Builds baseline/reference_cpu_flat.cpp against the reference's headers and the libraries in baseline/_ref
# (made by baseline/build_reference.sh) and runs it: the reference's own CPU kernels on the flat-gradient workload.
#   baseline/run_reference_cpu_flat.sh /path/to/stellatrain [numel] [steps]
set -euo pipefail
SRC=$(realpath "${1:?path to the reference tree}")
HERE=$(cd "$(dirname "$0")" && pwd)
PY=$(command -v python)
TORCH=$("$PY" -c 'import torch, os; print(os.path.dirname(torch.__file__))')
PYINC=$("$PY" -c 'import sysconfig; print(sysconfig.get_paths()["include"])')
OUT=${TMPDIR:-/tmp}/reference_cpu_flat
# same flags as the reference's own objects: -g -march=broadwell -O3 (backend/CMakeLists.txt:28-32)
/usr/bin/g++ -std=gnu++17 -g -O3 -march=broadwell -D_GLIBCXX_USE_CXX11_ABI=1 \
  -I"$SRC/backend/src" -I"$TORCH/include" -I"$TORCH/include/torch/csrc/api/include" -I"$PYINC" \
  "$HERE/reference_cpu_flat.cpp" -o "$OUT" \
  -L"$HERE/_ref" -lfasterdp_core -L"$TORCH/lib" -ltorch -ltorch_cpu -lc10 -ltorch_python -lpython3.12 \
  -Wl,-rpath,"$HERE/_ref" -Wl,-rpath,"$TORCH/lib" -Wl,--allow-shlib-undefined -pthread
LD_LIBRARY_PATH="$HERE/_ref:$TORCH/lib:${LD_LIBRARY_PATH:-}" "$OUT" "${@:2}"
