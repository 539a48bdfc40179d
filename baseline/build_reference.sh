#!/usr/bin/env bash
# Builds the UNMODIFIED reference (microsoft/mscclpp) natively with CMake into baseline/_ref, without network access.
#   usage: baseline/build_reference.sh [path to the reference checkout, default /root/reference]
# Its three external needs are met from what the image already has:
#   * nlohmann_json (FetchContent "json")  -> baseline/deps/json wraps a json.hpp found on the image
#   * libnuma                              -> baseline/deps/numa (two functions, built here as a static library)
#   * NVML                                 -> the toolkit's header and stub; the driver's library at run time
# InfiniBand, GDRCopy, tests and the Python bindings (nanobind / dlpack downloads) are switched off.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF_SRC="${1:-/root/reference}"
WORK="${TMPDIR:-/tmp}/mscclpp_ref_build_$$"
JSON_INC="$(python - <<'PY'
import glob, os, sysconfig
roots = [sysconfig.get_paths()["purelib"], "/usr/include", "/usr/local/include"]
for r in roots:
    for p in glob.glob(os.path.join(r, "**", "nlohmann", "json.hpp"), recursive=True):
        print(os.path.dirname(os.path.dirname(p)))
        raise SystemExit
PY
)"
[ -n "$JSON_INC" ] || { echo "no nlohmann/json.hpp on this image" >&2; exit 1; }
mkdir -p "$WORK/numa" "$WORK/src"
cp -r "$REF_SRC/." "$WORK/src/"          # the checkout may be read-only; nothing in the copy is edited
gcc -O2 -fPIC -c "$HERE/deps/numa/numa.c" -I "$HERE/deps/numa" -o "$WORK/numa/numa.o"
ar rcs "$WORK/numa/libnuma.a" "$WORK/numa/numa.o"
cp "$HERE/deps/numa/numa.h" "$WORK/numa/"
cmake -S "$WORK/src" -B "$WORK/build" -G Ninja -DCMAKE_BUILD_TYPE=Release \
  -DMSCCLPP_BYPASS_GPU_CHECK=ON -DMSCCLPP_USE_CUDA=ON -DMSCCLPP_GPU_ARCHS=100a \
  -DMSCCLPP_USE_IB=OFF -DMSCCLPP_USE_GDRCOPY=OFF -DMSCCLPP_BUILD_TESTS=OFF -DMSCCLPP_BUILD_PYTHON_BINDINGS=OFF \
  -DFETCHCONTENT_FULLY_DISCONNECTED=ON -DFETCHCONTENT_SOURCE_DIR_JSON="$HERE/deps/json" \
  -DNLOHMANN_JSON_INCLUDE_DIR="$JSON_INC" \
  -DNUMA_ROOT_DIR="$WORK/numa" -DNUMA_INCLUDE_DIR="$WORK/numa" -DNUMA_LIB_DIR="$WORK/numa" \
  -DCMAKE_CUDA_COMPILER="${CUDA_HOME:-/usr/local/cuda}/bin/nvcc"
cmake --build "$WORK/build" -j "$(nproc)"
cmake --install "$WORK/build" --prefix "$HERE/_ref"
# the reference's own execution plans (test inputs of its executor), for the plan-compatibility tests
mkdir -p "$HERE/_ref/share/execution-files"
cp "$REF_SRC"/test/execution-files/*.json "$HERE/_ref/share/execution-files/"
echo "installed: $HERE/_ref/lib"
