"""GGUF v3 files through the library's reader (csrc/gguf.cpp): the reference's `Gguf`
(src/gguf.rs) with the same names, validation rules and error kinds.  `InvalidData` for a
malformed directory, a missing tensor or key, an out-of-range row or expert; `UnexpectedEof`
for a positional read that the file can no longer satisfy."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _abi
from .gpu import Buffer, Gpu, InvalidData, IngotError, Matrix, Tensor, Weight


class UnexpectedEof(IngotError, EOFError):
    """io::ErrorKind::UnexpectedEof: the file ended before the bytes a tensor promised."""


class _Info(C.Structure):
    _fields_ = [("dims", C.c_uint64 * 4), ("rank", C.c_uint32), ("kind", C.c_uint32), ("offset", C.c_uint64),
                ("shard", C.c_uint32), ("reserved", C.c_uint32), ("stride", C.c_uint64), ("bytes", C.c_uint64)]

    def tensor(self) -> Tensor:
        return Tensor([int(self.dims[i]) for i in range(self.rank)], int(self.kind), int(self.offset), int(self.shard),
                      int(self.stride), int(self.bytes))


def _info_of(t: Tensor) -> _Info:
    info = _Info()
    for i, d in enumerate(t.dims):
        info.dims[i] = d
    info.rank, info.kind, info.offset, info.shard, info.stride, info.bytes = len(t.dims), t.kind, t.offset, t.shard, t.stride, t.bytes
    return info


class Gguf:
    """An opened model file (or the shards of a split model)."""

    def __init__(self, path: str):
        self._lib = _abi.load()
        h = C.c_void_p()
        self._h = None
        self._check(self._lib.ingot_gguf_open(str(path).encode(), C.byref(h)))
        self._h = h.value
        self.architecture = self._lib.ingot_gguf_architecture(self._h).decode()
        self.tensors: dict[str, Tensor] = {}
        name, info = C.c_char_p(), _Info()
        for i in range(self._lib.ingot_gguf_tensor_count(self._h)):
            self._check(self._lib.ingot_gguf_tensor_at(self._h, i, C.byref(name), C.byref(info)))
            self.tensors[name.value.decode()] = info.tensor()

    @staticmethod
    def open(path: str) -> "Gguf":
        return Gguf(path)

    def close(self) -> None:
        if self._h:
            self._lib.ingot_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int) -> None:
        if status == _abi.OK:
            return
        msg = self._lib.ingot_gguf_last_error().decode(errors="replace")
        if status == _abi.EOF:
            raise UnexpectedEof(msg)
        raise InvalidData(msg)

    @property
    def bytes_read(self) -> int:
        return int(self._lib.ingot_gguf_bytes_read(self._h))

    def tensor(self, name: str) -> Tensor:
        info = _Info()
        self._check(self._lib.ingot_gguf_tensor(self._h, name.encode(), C.byref(info)))
        return info.tensor()

    def integer(self, key: str) -> int:
        v = C.c_uint64()
        self._check(self._lib.ingot_gguf_integer(self._h, key.encode(), C.byref(v)))
        return int(v.value)

    def optional_integer(self, key: str):
        try:
            return self.integer(key)
        except InvalidData:
            return None

    def float(self, key: str) -> float:
        v = C.c_float()
        self._check(self._lib.ingot_gguf_float(self._h, key.encode(), C.byref(v)))
        return float(v.value)

    def string(self, key: str) -> str:
        v = C.c_char_p()
        self._check(self._lib.ingot_gguf_string(self._h, key.encode(), C.byref(v)))
        return v.value.decode()

    def integers(self, key: str) -> list[int]:
        n, v = C.c_uint64(), C.c_uint64()
        self._check(self._lib.ingot_gguf_array_length(self._h, key.encode(), C.byref(n)))
        out = []
        for i in range(n.value):
            self._check(self._lib.ingot_gguf_array_integer(self._h, key.encode(), i, C.byref(v)))
            out.append(int(v.value))
        return out

    def strings(self, key: str) -> list[str]:
        n, v = C.c_uint64(), C.c_char_p()
        self._check(self._lib.ingot_gguf_array_length(self._h, key.encode(), C.byref(n)))
        out = []
        for i in range(n.value):
            self._check(self._lib.ingot_gguf_array_string(self._h, key.encode(), i, C.byref(v)))
            out.append(v.value.decode())
        return out

    def read_range(self, t: Tensor, offset: int, length: int) -> np.ndarray:
        out = np.empty(length, np.uint8)
        info = _info_of(t)
        self._check(self._lib.ingot_gguf_read_range(self._h, C.byref(info), offset, out.ctypes.data, length))
        return out

    def rows(self, name: str, rows: list[int]) -> Matrix:
        """The listed rows in caller order (Gguf::rows)."""
        t = self.tensor(name)
        idx = np.asarray(rows, np.uint64)
        out = np.empty(max(len(rows), 1) * t.stride, np.uint8)
        self._check(self._lib.ingot_gguf_rows(self._h, name.encode(), idx.ctypes.data, len(rows), out.ctypes.data))
        return Matrix(out[:len(rows) * t.stride], t.dims[0], len(rows), 1, t.kind, t.stride)

    def matrix(self, name: str, shape: list[int], experts: list[int]) -> Matrix:
        """The listed experts of a tensor of exactly `shape` (Gguf::matrix)."""
        t = self.tensor(name)
        sh, ex = np.asarray(shape, np.uint64), np.asarray(experts, np.uint64)
        rows = shape[1] if len(shape) > 1 else 1
        out = np.empty(max(len(experts), 1) * t.stride * rows, np.uint8)
        self._check(self._lib.ingot_gguf_matrix(self._h, name.encode(), sh.ctypes.data, len(shape), ex.ctypes.data, len(experts),
                                                out.ctypes.data))
        return Matrix(out[:len(experts) * t.stride * rows], shape[0], rows, len(experts), t.kind, t.stride)

    def load_weight(self, gpu: Gpu, name: str, shape: list[int]) -> Weight:
        """Weight::load: shape check, then the tensor's bytes resident in HBM."""
        sh = np.asarray(shape, np.uint64)
        dev, info = C.c_void_p(), _Info()
        st = self._lib.ingot_weight_load(gpu._h, self._h, name.encode(), sh.ctypes.data, len(shape), C.byref(dev), C.byref(info))
        self._check(st)
        t = info.tensor()
        return Weight(Buffer(gpu, dev.value, t.bytes), t)
