#!/usr/bin/env bash
# Builds the UNMODIFIED reference (kaist-ina/stellatrain) out of tree and installs what its Python driver needs into
# baseline/_ref, for `bench.py --impl reference`.
#
#   baseline/build_reference.sh /path/to/stellatrain [build-dir]
#
# The reference is a CMake project (backend/CMakeLists.txt); `pip install` of its tree fails for want of a setup.py.
# Its sources are compiled as they are.  What the newer tool chain of this image needs (the reference was written for
# nvcr.io/nvidia/pytorch:23.06, Dockerfile:1) is supplied from outside, through a file given as CMAKE_PROJECT_INCLUDE:
#   * torch 2.11 headers need C++17 where the target asks for standard 14;
#   * <nvToolsExt.h> only exists as <nvtx3/nvToolsExt.h> in CUDA 12.9: a one-line forwarding header on the include path;
#   * core.cpp uses std::ofstream without <fstream>, which older libstdc++ headers pulled in: -include fstream;
#   * torch's include directory carries an older copy of the protobuf headers: the vendored ones are put first;
#   * pybind11's FindPython mode needs the Development.Module component.
# The system compiler is named explicitly: a wrapper compiler earlier on PATH linked libstdc++ statically into libzmq,
# whose copy of the iostream symbols then crashed the first `std::cerr << number` of the engine.
# Build type RelWithDebInfo (-g -O3) is what the reference's Dockerfile asks for (Dockerfile:27).
set -euo pipefail
SRC=$(realpath "${1:?path to the reference tree}")
WORK=${2:-/tmp/refbuild}
HERE=$(cd "$(dirname "$0")" && pwd)
PY=$(command -v python)
SITE=$("$PY" -c 'import torch, os; print(os.path.dirname(os.path.dirname(torch.__file__)))')
PYLIB=$(dirname "$SITE")                       # .../lib/python3.X
PYVER=$("$PY" -c 'import sys; print(f"{sys.version_info[0]}.{sys.version_info[1]}")')
PYINC=$("$PY" -c 'import sysconfig; print(sysconfig.get_paths()["include"])')

mkdir -p "$WORK/shim"
rm -rf "$WORK/backend" "$WORK/build"
cp -r "$SRC/backend" "$WORK/backend"           # the build writes generated protobuf sources next to the inputs
chmod -R u+w "$WORK/backend"
printf '#pragma once\n#include <nvtx3/nvToolsExt.h>\n' > "$WORK/shim/nvToolsExt.h"
cat > "$WORK/after_project.cmake" <<CMAKE
foreach(std 14 17)
  set(CMAKE_CXX\${std}_STANDARD_COMPILE_OPTION "-std=c++17;-include;fstream;-I$WORK/shim")
  set(CMAKE_CXX\${std}_EXTENSION_COMPILE_OPTION "-std=gnu++17;-include;fstream;-I$WORK/shim")
endforeach()
if(NOT COMMAND python_add_library)
  find_package(Python ${PYVER} COMPONENTS Interpreter Development.Module REQUIRED)
endif()
if(CMAKE_CURRENT_SOURCE_DIR STREQUAL CMAKE_SOURCE_DIR)
  include_directories(BEFORE \${CMAKE_SOURCE_DIR}/protobuf/src \${CMAKE_SOURCE_DIR}/protobuf/third_party/abseil-cpp)
endif()
CMAKE
COMPILERS=()
[ -x /usr/bin/g++ ] && COMPILERS=(-DCMAKE_C_COMPILER=/usr/bin/gcc -DCMAKE_CXX_COMPILER=/usr/bin/g++)
cmake -S "$WORK/backend" -B "$WORK/build" -G Ninja -DCMAKE_BUILD_TYPE=RelWithDebInfo -DCMAKE_POLICY_VERSION_MINIMUM=3.5 \
  -DCMAKE_PROJECT_INCLUDE="$WORK/after_project.cmake" -DPython_EXECUTABLE="$PY" "${COMPILERS[@]}" \
  -DCMAKE_PREFIX_PATH="$SITE/torch/share/cmake/Torch" -DPYTHON_LIB_PATH="$PYLIB" -DPYTHON_INCLUDE_PATH="$PYINC" \
  -DPYTHON_VERSION="$PYVER"
ninja -C "$WORK/build" fasterdp

DEST="$HERE/_ref"
rm -rf "$DEST"
mkdir -p "$DEST"
cp "$WORK"/build/fasterdp*.so "$DEST/"
# shared libraries the module needs at run time (found through LD_LIBRARY_PATH=baseline/_ref)
find "$WORK/build" -name '*.so*' ! -name 'fasterdp*.so' ! -name 'libprotoc*' \( -type f -o -type l \) -exec cp -P {} "$DEST/" \;
cp "$SRC/backend/src/python/fasterdp/model_wrapper.py" "$DEST/"
strip --strip-debug "$DEST"/*.so* 2>/dev/null || true
du -sh "$DEST"
