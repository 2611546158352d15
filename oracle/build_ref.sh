#!/bin/sh
# Compiles the reference's own scalar block decoders (weight_at, mix_weight_at,
# kquant_scale_min and the tables they name) as C++ into
# oracle/_ref/libref_decode.so.  The shader text is streamed from the reference
# tree into the compiler; none of it is written into this repository.
#   kernels/quant_tables.metal  (whole file, minus its two include lines)
#   kernels/iq3_mix.metal:6-36  (mix_half .. mix_weight_at)
#   kernels/moe.metal:6-89      (half_at, weight_at)
# usage: build_ref.sh <path of the reference tree>   (or INGOT_REFERENCE in the environment)
set -e
REF="${1:-$INGOT_REFERENCE}"
if [ -z "$REF" ] || [ ! -d "$REF/kernels" ]; then
  echo "usage: $0 <path of the reference tree>" >&2
  exit 2
fi
HERE="$(cd "$(dirname "$0")" && pwd)"
mkdir -p "$HERE/_ref"
{
  echo '#include "metal_shim.h"'
  sed -n '4,$p' "$REF/kernels/quant_tables.metal"
  sed -n '6,36p' "$REF/kernels/iq3_mix.metal"
  sed -n '6,89p' "$REF/kernels/moe.metal"
  cat "$HERE/ref_exports.inc"
} | g++ -x c++ -std=c++17 -O1 -ffp-contract=off -fno-fast-math -fPIC -shared \
        -I"$HERE" -Wno-attributes -o "$HERE/_ref/libref_decode.so" -
echo "built $HERE/_ref/libref_decode.so"
