"""Generates tests/golden/decode_kind*.npz.

Run in a container where the reference tree is mounted and oracle/_ref has
been built (`make -C oracle`).  For every format on the path it draws a few
rows of blocks (random ones plus edge cases: zero, subnormal and largest f16
scales, all-zero and all-ones quants) and stores

    raw        the GGUF bytes
    expected   the float32 bit patterns produced by the REFERENCE's own
               weight_at (kernels/moe.metal:11-89, kernels/iq3_mix.metal:17-36)
               compiled as C++ (oracle/build_ref.sh)
    gguf_equal whether gguf-py's NumPy dequantiser gave the same bits
               (quantised formats only)

The fixtures travel to machines without the reference tree, where the oracle
and the CUDA kernels are checked against them.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from ingot_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402

COLS, ROWS = 512, 6
EDGE_SCALES = [0x0000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0x3C00, 0x8001, 0xBC00]   # f16 bit patterns


def edge_cases(kind: int, raw: np.ndarray) -> None:
    """Overwrites the first blocks of `raw` [n_blocks, bytes] with edge cases."""
    n = raw.shape[0]
    scale_at = {synth.Q4_K: [0, 2], synth.Q6_K: [208], synth.Q4_0: [0], synth.Q8_0: [0]}.get(kind)
    if scale_at is None:
        return
    for i, bits in enumerate(EDGE_SCALES):
        if i >= n:
            break
        for off in scale_at:
            raw[i, off] = bits & 0xFF
            raw[i, off + 1] = bits >> 8
    if n > len(EDGE_SCALES) + 2:
        body = {synth.Q4_K: slice(4, 144), synth.Q6_K: slice(0, 208), synth.Q4_0: slice(2, 18),
                synth.Q8_0: slice(2, 34)}[kind]
        raw[len(EDGE_SCALES), body] = 0x00
        raw[len(EDGE_SCALES) + 1, body] = 0xFF
        if kind == synth.Q8_0:
            raw[len(EDGE_SCALES) + 2, body] = 0x80        # int8 -128


def main() -> None:
    if not O.ref_available():
        raise SystemExit("oracle/_ref/libref_decode.so is missing: run `make -C oracle` with the reference mounted")
    try:
        import gguf
        from gguf import quants
        gmap = {synth.Q4_0: gguf.GGMLQuantizationType.Q4_0, synth.Q8_0: gguf.GGMLQuantizationType.Q8_0,
                synth.Q4_K: gguf.GGMLQuantizationType.Q4_K, synth.Q6_K: gguf.GGMLQuantizationType.Q6_K}
    except Exception:   # gguf-py is optional
        quants, gmap = None, {}
    for kind in (synth.F32, synth.F16, synth.BF16, synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K):
        block, size = synth.geometry(kind)
        rng = np.random.default_rng(1000 + kind)
        raw = synth.random_blocks(kind, COLS // block * ROWS, rng)
        edge_cases(kind, raw)
        flat = np.ascontiguousarray(raw).reshape(-1)
        expected = O.ref_dequant(flat, COLS, ROWS, kind)
        gguf_equal = -1
        if kind in gmap:
            g = quants.dequantize(flat.reshape(ROWS, -1), gmap[kind]).astype(np.float32)
            gguf_equal = int(np.array_equal(g.view(np.uint32), expected.view(np.uint32)))
        path = os.path.join(HERE, f"decode_kind{kind}.npz")
        np.savez_compressed(path, raw=flat, cols=COLS, rows=ROWS, kind=kind,
                            expected_bits=expected.view(np.uint32), gguf_equal=gguf_equal)
        print(f"kind {kind}: {flat.size} bytes -> {expected.size} values, gguf_equal={gguf_equal}")


if __name__ == "__main__":
    main()
