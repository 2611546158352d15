"""The GGUF v3 reader against the reference's own micro-fixtures (src/gguf.rs:506-600,
src/weights.rs:104-131): directory validation, positional reads, rows and matrices, split
shards, truncation after opening.  CPU only, except the last test, which loads a tensor
into HBM and multiplies with it."""
import os
import struct

import numpy as np
import pytest

from ingot_b200 import InvalidData
from ingot_b200.gguf import Gguf, UnexpectedEof


def text(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def kv_text(key: str, value: str) -> bytes:
    return text(key) + struct.pack("<I", 8) + text(value)


def kv_u32(key: str, value: int) -> bytes:
    return text(key) + struct.pack("<II", 4, value)


def tensor_entry(name: str, dims, kind: int, offset: int) -> bytes:
    return text(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", kind, offset)


def build(kvs, tensors, payload: bytes, alignment: int = 32, version: int = 3, magic: int = 0x46554747) -> bytes:
    head = struct.pack("<IIQQ", magic, version, len(tensors), len(kvs)) + b"".join(kvs) + b"".join(tensors)
    head += b"\0" * (-len(head) % alignment)
    return head + payload


def f32(values) -> bytes:
    return np.asarray(values, np.float32).tobytes()


@pytest.fixture
def fixture_path(tmp_path):
    # the reference's "weight" fixture: one F32 tensor [2, 2] = 1, 2, 3, 4 (src/gguf.rs:517-541)
    p = tmp_path / "fixture.gguf"
    p.write_bytes(build([kv_text("general.architecture", "fixture")], [tensor_entry("weight", [2, 2], 0, 0)], f32([1, 2, 3, 4])))
    return p


def test_directory_and_positional_reads(fixture_path):
    g = Gguf.open(fixture_path)
    assert g.architecture == "fixture"
    t = g.tensor("weight")
    assert (t.dims, t.kind, t.stride, t.bytes, t.shard) == ([2, 2], 0, 8, 16, 0)
    assert t.offset % 32 == 0
    assert g.rows("weight", [1]).data.tobytes() == f32([3, 4])
    before = g.bytes_read
    m = g.rows("weight", [1, 0, 1, 0])                       # repeated indices keep caller order
    assert m.data.tobytes() == f32([3, 4, 1, 2, 3, 4, 1, 2]) and (m.cols, m.rows, m.count, m.stride) == (2, 4, 1, 8)
    assert g.bytes_read - before == 32
    before = g.bytes_read
    for bad in ([], [0, 2]):
        with pytest.raises(InvalidData):
            g.rows("weight", bad)
    assert g.bytes_read == before
    with pytest.raises(InvalidData):
        g.tensor("missing")
    assert g.read_range(t, 4, 8).tobytes() == f32([2, 3])
    with pytest.raises(InvalidData):
        g.read_range(t, 12, 8)                              # beyond the tensor
    assert g.string("general.architecture") == "fixture"
    with pytest.raises(InvalidData):
        g.integer("general.architecture")


def test_truncation_after_opening_is_unexpected_eof(fixture_path):
    g = Gguf.open(fixture_path)
    size = os.path.getsize(fixture_path)
    with open(fixture_path, "r+b") as f:
        f.truncate(size - 6)                                # payload + 10 bytes remain, as in src/gguf.rs:575
    with pytest.raises(UnexpectedEof):
        g.rows("weight", [1])
    before = g.bytes_read
    with pytest.raises(UnexpectedEof):
        g.rows("weight", [0, 1, 0, 1])
    assert g.bytes_read - before == 16                      # every row is attempted; the two valid ones count
    with pytest.raises(InvalidData):                        # reopening validates the directory against the new size
        Gguf.open(fixture_path)


def test_truncated_and_malformed_headers(tmp_path):
    def opens(data: bytes):
        p = tmp_path / "bad.gguf"
        p.write_bytes(data)
        return Gguf.open(p)
    arch = [kv_text("general.architecture", "fixture")]
    one = [tensor_entry("weight", [2, 2], 0, 0)]
    with pytest.raises(InvalidData):
        opens(b"GGUF\x03\0\0\0")                            # src/gguf.rs:506-512
    with pytest.raises(InvalidData):
        opens(build(arch, one, f32([1, 2, 3, 4]), version=2))
    with pytest.raises(InvalidData):
        opens(build(arch, one, f32([1, 2, 3, 4]), magic=0x46554746))
    with pytest.raises(InvalidData):
        opens(build([], one, f32([1, 2, 3, 4])))            # missing architecture
    with pytest.raises(InvalidData):
        opens(build(arch + arch, one, f32([1, 2, 3, 4])))   # duplicate metadata
    with pytest.raises(InvalidData):
        opens(build(arch, one + one, f32([1, 2, 3, 4])))    # duplicate tensor
    with pytest.raises(InvalidData):
        opens(build(arch, one, f32([1, 2, 3])))             # extends beyond file
    with pytest.raises(InvalidData):
        opens(build(arch, [tensor_entry("a", [2, 2], 0, 0), tensor_entry("b", [2, 2], 0, 0)], f32(range(8))))    # overlap
    with pytest.raises(InvalidData):
        opens(build(arch, [tensor_entry("w", [2, 2], 0, 8)], b"\0" * 8 + f32([1, 2, 3, 4])))                      # offset not aligned
    with pytest.raises(InvalidData):
        opens(build(arch, [tensor_entry("w", [100, 2], 12, 0)], b"\0" * 1000))                                    # 100 is not a whole Q4_K block
    with pytest.raises(InvalidData):
        opens(build(arch, [tensor_entry("w", [2, 2], 19, 0)], f32([1, 2, 3, 4])))                                 # unknown GGML type
    with pytest.raises(InvalidData):
        opens(build(arch, [tensor_entry("w", [2, 0], 0, 0)], b""))                                                # zero dimension
    with pytest.raises(InvalidData):
        opens(build(arch, [tensor_entry("w", [2, 1, 1, 1, 1], 0, 0)], f32([1, 2])))                               # rank 5
    with pytest.raises(InvalidData):
        opens(build(arch + [kv_u32("general.alignment", 24)], one, f32([1, 2, 3, 4]), alignment=24))              # not a power of two
    nested = text("a") + struct.pack("<II", 9, 9) + struct.pack("<Q", 0)
    with pytest.raises(InvalidData):
        opens(build(arch + [nested], one, f32([1, 2, 3, 4])))
    g = opens(build(arch + [kv_u32("general.alignment", 64)], one, f32([1, 2, 3, 4]), alignment=64))
    assert g.tensor("weight").offset % 64 == 0 and g.integer("general.alignment") == 64


def test_metadata_values_and_arrays(tmp_path):
    arr_i = text("tokenizer.ids") + struct.pack("<IIQ", 9, 4, 3) + struct.pack("<III", 7, 8, 9)
    arr_s = text("tokenizer.tokens") + struct.pack("<IIQ", 9, 8, 2) + text("a") + text("bc")
    kvs = [kv_text("general.architecture", "fixture"), text("x.eps") + struct.pack("<If", 6, 1e-6),
           text("x.big") + struct.pack("<IQ", 10, 1 << 40), text("x.flag") + struct.pack("<IB", 7, 1), arr_i, arr_s]
    p = tmp_path / "meta.gguf"
    p.write_bytes(build(kvs, [tensor_entry("weight", [2, 2], 0, 0)], f32([1, 2, 3, 4])))
    g = Gguf.open(p)
    assert g.integer("x.big") == 1 << 40 and g.integer("x.flag") == 1
    assert abs(g.float("x.eps") - 1e-6) < 1e-12
    assert g.integers("tokenizer.ids") == [7, 8, 9] and g.strings("tokenizer.tokens") == ["a", "bc"]
    assert g.optional_integer("nope") is None
    with pytest.raises(InvalidData):
        g.strings("tokenizer.ids")


def test_expert_matrix_and_split_shards(tmp_path):
    # src/weights.rs:104-131: experts [2, 2, 4] F32, expert e holds 10 e + 1..4
    payload = b"".join(f32([e * 10 + v for v in range(1, 5)]) for e in range(4))
    p = tmp_path / "experts.gguf"
    p.write_bytes(build([kv_text("general.architecture", "fixture")], [tensor_entry("experts", [2, 2, 4], 0, 0)], payload))
    g = Gguf.open(p)
    m = g.matrix("experts", [2, 2, 4], [3, 0])
    assert (m.cols, m.rows, m.count) == (2, 2, 2) and m.data.tobytes() == f32([31, 32, 33, 34, 1, 2, 3, 4])
    for shape, experts in (([2, 2, 3], [0]), ([2, 2, 4], []), ([2, 2, 4], [4])):
        with pytest.raises(InvalidData):
            g.matrix("experts", shape, experts)
    # a two-shard model: the primary shard names the second one
    base = [kv_text("general.architecture", "fixture"), kv_u32("split.count", 2), kv_u32("split.tensors.count", 2)]
    a = tmp_path / "m-00001-of-00002.gguf"
    b = tmp_path / "m-00002-of-00002.gguf"
    a.write_bytes(build(base + [kv_u32("split.no", 0)], [tensor_entry("w0", [2, 2], 0, 0)], f32([1, 2, 3, 4])))
    b.write_bytes(build(base + [kv_u32("split.no", 1)], [tensor_entry("w1", [2, 1], 0, 0)], f32([5, 6])))
    g = Gguf.open(a)
    assert sorted(g.tensors) == ["w0", "w1"] and g.tensor("w1").shard == 1
    assert g.rows("w1", [0]).data.tobytes() == f32([5, 6])
    with pytest.raises(InvalidData):
        Gguf.open(b)                                        # pass the primary shard
    b.write_bytes(build(base + [kv_u32("split.no", 1)], [tensor_entry("w0", [2, 1], 0, 0)], f32([5, 6])))
    with pytest.raises(InvalidData):
        Gguf.open(a)                                        # duplicate tensor across shards


@pytest.mark.gpu
def test_weight_load_uploads_and_projects(gpu, tmp_path):
    # the reference's fixture (src/metal/tests.rs:1887-1917): F32 experts [2, 2, 4]; x = [1, 1], ids [0, 1] -> [3, 7, 23, 27]
    from ingot_b200 import Q4_K, synth
    from oracle import oracle as O
    payload = b"".join(f32([e * 10 + v for v in range(1, 5)]) for e in range(4))
    raw = synth.random_matrix(Q4_K, 512, 40, seed=4)
    pad = b"\0" * (-len(payload) % 32)
    p = tmp_path / "load.gguf"
    p.write_bytes(build([kv_text("general.architecture", "fixture")],
                        [tensor_entry("experts", [2, 2, 4], 0, 0), tensor_entry("blk.0.attn_q.weight", [512, 40], 12, len(payload) + len(pad))],
                        payload + pad + raw.tobytes()))
    g = Gguf.open(p)
    w = g.load_weight(gpu, "experts", [2, 2, 4])
    w.require_f32()
    ids = gpu.bytes(np.array([0, 1], np.uint32))
    y = gpu.output(4)
    assert gpu.generic_routed(None, w, [gpu.floats(np.ones(2, np.float32)), ids, y], False, 2, 2)
    assert gpu.finish(None, y).tolist() == [3.0, 7.0, 23.0, 27.0]
    with pytest.raises(InvalidData):
        g.load_weight(gpu, "experts", [2, 2, 3])
    q = g.load_weight(gpu, "blk.0.attn_q.weight", [512, 40])
    x = synth.activations(1, 512, seed=5)
    got = gpu.finish(None, q.project(gpu, None, gpu.floats(x)))
    e = O.matvec_f64(raw, 512, 40, Q4_K, x)[0]
    assert (np.abs(got - e) <= 1e-4 * max(1.0, float(np.sqrt(np.mean(e * e)))) + 5e-5 * np.abs(e)).all()
