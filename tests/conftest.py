"""Shared test configuration: the `gpu` marker, repo paths on sys.path, and the
fixtures that reproduce the reference's own synthetic test inputs."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with `-m gpu` on the GPU box")


def tol_ref(expected: np.ndarray) -> np.ndarray:
    """The reference's own bound for a GEMV against an f64 dot of the dequantised
    weights: |a - e| <= 1e-4 + 5e-5 |e| (tests/projections.rs:42-46)."""
    return 1e-4 + 5e-5 * np.abs(expected)


def tol_ref_scaled(expected: np.ndarray) -> np.ndarray:
    """tol_ref with its absolute part scaled by the output RMS (when above 1): the reference's
    bound was written for model weights with O(1) outputs; the synthetic benchmark blocks give
    outputs of magnitude ~300, where fp32 accumulation alone exceeds 1e-4 absolute."""
    rms = float(np.sqrt(np.mean(np.square(expected)))) if expected.size else 0.0
    return 1e-4 * max(1.0, rms) + 5e-5 * np.abs(expected)


def tol_contract(expected: np.ndarray) -> np.ndarray:
    """The stated contract: 1e-3 relative / 1e-4 absolute.  The absolute part is
    scaled by the output's RMS when that exceeds 1, because the synthetic
    benchmark weights give outputs of magnitude ~300 where 1e-4 absolute is
    below fp32 resolution of the sum."""
    rms = float(np.sqrt(np.mean(np.square(expected)))) if expected.size else 0.0
    return 1e-4 * max(1.0, rms) + 1e-3 * np.abs(expected)


def standard_x(n: int) -> np.ndarray:
    """x[i] = ((i*17 % 31) - 15) / 32, the reference's usual activation pattern
    (tests/projections.rs:32-34)."""
    i = np.arange(n, dtype=np.int64)
    return (((i * 17) % 31) - 15).astype(np.float32) * np.float32(0.03125)


class Lcg:
    """The reference bench's generator: s = s*6364136223846793005 +
    1442695040888963407; u = (s >> 11) / 2^53 (src/expert_bench.rs:5-10)."""

    def __init__(self, seed: int):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def next(self) -> float:
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return (self.s >> 11) / float(1 << 53)


def lcg_q4k_fixture(cols: int = 2560, rows: int = 37, experts: int = 3, seed: int = 23) -> np.ndarray:
    """Random Q4_K bytes the way src/expert_bench.rs:652-688 draws them: every byte
    u*256, then the two f16 scales of each 144-byte block set to 0x1c00 + u*2560."""
    g = Lcg(seed)
    n = cols // 256 * 144 * rows * experts
    data = np.empty(n, dtype=np.uint8)
    for i in range(n):
        data[i] = int(g.next() * 256.0) & 0xFF
    for b in range(n // 144):
        for off in (0, 2):
            bits = 0x1C00 + int(g.next() * 2560.0)
            data[b * 144 + off] = bits & 0xFF
            data[b * 144 + off + 1] = bits >> 8
    return data


def q4_0_hand_fixture(rows: int = 7, cols: int = 64, experts: int = 5) -> np.ndarray:
    """The hand-built Q4_0 fixture of src/metal/tests.rs:42-51: scale 0.5 (0x3800),
    byte j of a block = ((row+block+j+3)%16) << 4 | ((row+block+j)%16)."""
    out = bytearray()
    for row in range(rows * experts):
        for block in range(cols // 32):
            out += (0x3800).to_bytes(2, "little")
            for j in range(16):
                out.append((((row + block + j + 3) % 16) << 4 | ((row + block + j) % 16)) & 0xFF)
    return np.frombuffer(bytes(out), dtype=np.uint8).copy()


def q4_0_hand_expected(ids, rows, cols, top, per_pair, inputs):
    """Closed-form expectation of the same test (src/metal/tests.rs:73-88), in f64."""
    pairs = len(ids)
    out = np.zeros((pairs, rows), dtype=np.float64)
    j = np.arange(cols)
    for pair in range(pairs):
        for r in range(rows):
            row = int(ids[pair]) * rows + r
            nib = (row + j // 32 + j % 16 + np.where(j % 32 >= 16, 3, 0)) % 16
            inp = pair if per_pair else pair // top
            out[pair, r] = np.sum((nib.astype(np.float64) - 8.0) * 0.5 * inputs[inp * cols:(inp + 1) * cols].astype(np.float64))
    return out


@pytest.fixture(scope="session")
def gpu():
    from ingot_b200 import Gpu
    g = Gpu(0)
    yield g
    g.close()
