#!/usr/bin/env bash
# Builds libframe_b200_hal.so: the C++20 adapter that plugs libframe_b200 (C ABI) into a Frame
# process as backend "cuda" (hal::Backend + one KernelFn per op + the new-op registrations).
# It compiles against the Frame headers and leaves Frame's own symbols undefined: they are
# resolved at load time by the Frame build of the host process (a Frame built with
# FRAME_ENABLE_CUDA=OFF), exactly like any other backend plugin.
#
#   usage: frame_public_b200/host/build_adapter.sh FRAME_ROOT     (or set FRAME_REFERENCE_ROOT)
set -euo pipefail
FRAME_ROOT="${1:-${FRAME_REFERENCE_ROOT:-}}"
if [ -z "$FRAME_ROOT" ]; then
  echo "usage: build_adapter.sh FRAME_ROOT   (or set FRAME_REFERENCE_ROOT): the root of a Frame source tree" >&2
  exit 2
fi
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
PKG="$(dirname "$HERE")"
ROOT="$(dirname "$PKG")"
if [ ! -d "$FRAME_ROOT/include/frame" ]; then
  echo "build_adapter.sh: Frame headers not found under $FRAME_ROOT (the prebuilt adapter is used as it is)" >&2
  exit 0
fi
mkdir -p "$PKG/lib"
${CXX:-g++} -std=c++20 -O2 -ffp-contract=off -fPIC -shared \
  -I"$FRAME_ROOT/include" -I"$ROOT/include" -I"$HERE" \
  "$HERE/b200_backend.cpp" "$HERE/b200_kernels.cpp" "$HERE/new_ops.cpp" \
  -o "$PKG/lib/libframe_b200_hal.so" \
  -L"$PKG/lib" -lframe_b200 -Wl,-rpath,'$ORIGIN' -Wl,--version-script="$HERE/adapter_exports.map"
echo "built $PKG/lib/libframe_b200_hal.so"
