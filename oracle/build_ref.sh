#!/usr/bin/env bash
# TEST INFRASTRUCTURE — builds the reference's own CPU implementation of the
# compiled-graph path from the reference's sources, where they lie, into
# oracle/_ref/ (git-ignored).  Nothing is copied from the reference tree; only
# object files and one shared library are produced.
#
#   usage: oracle/build_ref.sh [REFERENCE_ROOT]      (default FRAME_ROOT)
#
# Product of this script:
#   oracle/_ref/libframe_ref.so   core + ir + ops + schemas + compiler + passes +
#                                 runtime + nn + backends/cpu of the reference,
#                                 object files linked directly so that the
#                                 static op / kernel / backend registrars run at
#                                 load time (the reference links its archives
#                                 WHOLE for the same reason).
#   oracle/_ref/libframe_ref_shim.so  the extern "C" shim of oracle/ref_shim.cpp.
#   oracle/_ref/_core.*.so        the reference's own pybind11 module (python/src/*.cpp, compiled
#                                 where they lie) linked against libframe_ref.so: the reference's
#                                 Python surface (Tensor.to, compile, Executable.run), used by the
#                                 GPU tests to drive this repository's backend from Python.  Skipped
#                                 with a note when pybind11 is not importable.
#
# Flags: -O2 -ffp-contract=off, no -march=native, no -ffast-math, so that
# `acc += a*b` is never contracted into an FMA and the numbers equal those of
# the reference's own Debug/Release builds.
# src/backends/cpu/kernels/fft.cpp is skipped: it needs pocketfft, which the
# reference downloads at configure time; rfft/irfft are not on the path.
set -euo pipefail
REF="${1:-${FRAME_REFERENCE_ROOT:-}}"
if [ -z "$REF" ]; then
  echo "usage: oracle/build_ref.sh FRAME_ROOT   (or set FRAME_REFERENCE_ROOT): the root of a Frame source tree" >&2
  exit 2
fi
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
OBJ="$OUT/obj"
mkdir -p "$OBJ"

if [ ! -d "$REF/src" ]; then
  echo "build_ref.sh: reference tree not found at $REF (prebuilt files in $OUT are used as they are)" >&2
  exit 0
fi

CXX="${CXX:-g++}"
CXXFLAGS="-std=c++20 -O2 -ffp-contract=off -fPIC -fvisibility=default -I$REF/include -I$REF/src"
DIRS="core ir ops ops/schemas compiler compiler/passes runtime nn data interop backends/cpu backends/cpu/kernels"

list_sources() {
  for d in $DIRS; do
    for f in "$REF/src/$d"/*.cpp; do
      [ -e "$f" ] || continue
      case "$f" in */backends/cpu/kernels/fft.cpp) continue ;; esac
      echo "$f"
    done
  done
}

compile_one() {
  src="$1"
  rel="${src#$REF/src/}"
  obj="$OBJ/$(echo "${rel%.cpp}" | tr '/' '_').o"
  if [ ! -e "$obj" ] || [ "$src" -nt "$obj" ]; then
    $CXX $CXXFLAGS -c "$src" -o "$obj"
  fi
}
export -f compile_one
export REF OBJ CXX CXXFLAGS

list_sources | xargs -P "$(nproc)" -I{} bash -c 'compile_one "$@"' _ {}

$CXX -shared -o "$OUT/libframe_ref.so" "$OBJ"/*.o -lpthread -Wl,--version-script="$HERE/ref_exports.map"
$CXX $CXXFLAGS -shared -o "$OUT/libframe_ref_shim.so" "$HERE/ref_shim.cpp" \
  -L"$OUT" -lframe_ref -Wl,-rpath,'$ORIGIN' -Wl,--version-script="$HERE/shim_exports.map"
echo "built $OUT/libframe_ref.so and libframe_ref_shim.so"

# ---- the reference's Python bindings -----------------------------------------------------------
PY="${PYTHON:-python}"
if PYBIND_INC="$($PY -c 'import pybind11; print(pybind11.get_include())' 2>/dev/null)"; then
  PY_INC="$($PY -c 'import sysconfig; print(sysconfig.get_paths()["include"])')"
  EXT="$($PY -c 'import sysconfig; print(sysconfig.get_config_var("EXT_SUFFIX"))')"
  PYOBJ="$OUT/pyobj"
  mkdir -p "$PYOBJ"
  compile_py() {
    src="$1"
    obj="$PYOBJ/$(basename "${src%.cpp}").o"
    if [ ! -e "$obj" ] || [ "$src" -nt "$obj" ]; then
      $CXX $CXXFLAGS -fvisibility=hidden -I"$PYBIND_INC" -I"$PY_INC" -I"$REF/python/src" -c "$src" -o "$obj"
    fi
  }
  export -f compile_py
  export PYOBJ PYBIND_INC PY_INC
  ls "$REF"/python/src/*.cpp | xargs -P "$(nproc)" -I{} bash -c 'compile_py "$@"' _ {}
  $CXX -shared -o "$OUT/_core$EXT" "$PYOBJ"/*.o -L"$OUT" -lframe_ref -Wl,-rpath,'$ORIGIN'
  echo "built $OUT/_core$EXT"
else
  echo "build_ref.sh: pybind11 not importable, the reference's Python bindings are not built" >&2
fi
