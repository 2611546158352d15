"""Seeded synthetic block-quantised tensors with the shapes, block formats and
value distributions of the benchmark configurations.

Real GGUF model files are not available offline; these stand in for them.
Only raw bytes are produced (the GGUF on-disk block layout); nothing here
decodes them.
"""
from __future__ import annotations

import numpy as np

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K, BF16 = 0, 1, 2, 8, 12, 14, 30

# (block elements, block bytes); the reference's geometry(): src/gguf.rs:470-491
GEOMETRY = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_0: (32, 18), Q8_0: (32, 34),
            Q4_K: (256, 144), Q6_K: (256, 210)}


def geometry(kind: int) -> tuple[int, int]:
    try:
        return GEOMETRY[kind]
    except KeyError:
        raise ValueError(f"GGML type {kind} is unsupported") from None


def stride_of(kind: int, cols: int) -> int:
    block, size = geometry(kind)
    if cols <= 0 or cols % block:
        raise ValueError("cols is not a whole number of blocks")
    return cols // block * size


def _f16_bits(values: np.ndarray) -> np.ndarray:
    return values.astype(np.float16).view(np.uint16)


def random_blocks(kind: int, n_blocks: int, rng: np.random.Generator) -> np.ndarray:
    """uint8 [n_blocks, block_bytes] drawn like the benchmark configurations:
    quant bytes and packed scale bytes uniform; f16 super-scales |N(0, s)|."""
    _, size = geometry(kind)
    # uniform bytes, drawn four at a time (full-range 32-bit draws are the generator's fast path)
    n = n_blocks * size
    raw = rng.integers(0, 1 << 32, size=(n + 3) // 4, dtype=np.uint32).view(np.uint8)[:n].reshape(n_blocks, size)
    if kind == Q4_K:      # [f16 d][f16 dmin][12 scales][128 qs]
        raw[:, 0:2] = _f16_bits(np.abs(rng.normal(0.0, 0.02, n_blocks))).reshape(-1, 1).view(np.uint8)
        raw[:, 2:4] = _f16_bits(np.abs(rng.normal(0.0, 0.01, n_blocks))).reshape(-1, 1).view(np.uint8)
    elif kind == Q6_K:    # [128 ql][64 qh][16 int8 scales][f16 d]
        raw[:, 208:210] = _f16_bits(np.abs(rng.normal(0.0, 0.02, n_blocks)) / 32.0).reshape(-1, 1).view(np.uint8)
    elif kind == Q4_0:    # [f16 d][16 qs]
        raw[:, 0:2] = _f16_bits(np.abs(rng.normal(0.0, 0.02, n_blocks))).reshape(-1, 1).view(np.uint8)
    elif kind == Q8_0:    # [f16 d][32 int8]
        raw[:, 0:2] = _f16_bits(np.abs(rng.normal(0.0, 0.02, n_blocks)) / 8.0).reshape(-1, 1).view(np.uint8)
    elif kind == F32:
        raw = rng.normal(0.0, 0.05, n_blocks).astype(np.float32).view(np.uint8).reshape(n_blocks, 4)
    elif kind == F16:
        raw = rng.normal(0.0, 0.05, n_blocks).astype(np.float16).view(np.uint8).reshape(n_blocks, 2)
    elif kind == BF16:
        bits = rng.normal(0.0, 0.05, n_blocks).astype(np.float32).view(np.uint32)
        raw = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16).view(np.uint8).reshape(n_blocks, 2)
    return raw


def random_matrix(kind: int, cols: int, rows: int, count: int = 1, seed: int = 0) -> np.ndarray:
    """Flat uint8 array of `count` stacked experts of rows x stride bytes."""
    block, _ = geometry(kind)
    rng = np.random.default_rng(seed)
    return random_blocks(kind, cols // block * rows * count, rng).reshape(-1)


def activations(tokens: int, cols: int, seed: int = 0) -> np.ndarray:
    """float32 N(0,1) [tokens, cols]."""
    return np.random.default_rng(seed).normal(0.0, 1.0, (tokens, cols)).astype(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- model shapes of the benchmark configurations ---------------------------

def qwen3_8b_layer() -> list[tuple[str, int, int, int]]:
    """(role, cols K, rows N, kind) of one Qwen3-8B Q4_K_M decoder layer."""
    return [("q", 4096, 4096, Q4_K), ("k", 4096, 1024, Q4_K), ("v", 4096, 1024, Q6_K),
            ("o", 4096, 4096, Q4_K), ("gate", 4096, 12288, Q4_K), ("up", 4096, 12288, Q4_K),
            ("down", 12288, 4096, Q6_K)]


QWEN3_8B = {"layers": 36, "hidden": 4096, "ffn": 12288, "vocab": 151936, "head_kind": Q6_K}
GEMMA3_4B = {"layers": 34, "hidden": 2560, "q": 2048, "kv": 1024, "ffn": 10240, "vocab": 262144, "kind": Q4_0}
QWEN3_30B_A3B = {"layers": 48, "hidden": 2048, "experts": 128, "top": 8, "ffn": 768, "kind": Q4_K}
