"""Host-side mirror of the reference's operator interface over the C ABI.

Names, argument meaning and error behaviour follow the reference's Rust types
so that tests read like the reference's own:

  Gpu, Buffer, Command   src/metal.rs (Gpu::bytes/floats/output/matvec/matmul/
                         op/activation/merge/dequant/project/finish/read_u32)
  generic_* operators    src/metal_generic.rs:175-329
  Tensor, Matrix         src/gguf.rs:18-25, 462-469
  Weight                 src/weights.rs:10-45

Errors: `InvalidData` (io::ErrorKind::InvalidData), `DeviceError`
(io::Error::other, sticky), `DeviceTimeout`.  Operators without a kernel for a
type return None / False like the reference's Ok(None) / Ok(false).
Everything runs through libingot_cuda.so; nothing is computed on the host.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _abi
from .synth import geometry, stride_of

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K, BF16 = 0, 1, 2, 8, 12, 14, 30
X_PACKED = _abi.X_PACKED     # x_kind of rows produced by Gpu.pack_x
X_PACKED_HI = _abi.X_PACKED_HI   # x_kind of rows produced by Gpu.pack_x_hi (bfloat16 activations, up to eight tokens per pass)
X_DIGITS = _abi.X_DIGITS     # x_kind of rows produced by Gpu.pack_digits (tcgen05 int8 GEMV)


class IngotError(Exception):
    pass


class InvalidData(IngotError, ValueError):
    """Shape, layout, bounds or unsupported-format error."""


class DeviceError(IngotError, RuntimeError):
    """CUDA failure; the handle must be recreated ("requires reload")."""


class DeviceTimeout(IngotError, TimeoutError):
    """A bounded device-side wait ran out."""


@dataclass
class Tensor:
    """A tensor descriptor: dims[0] = cols (contiguous), dims[1] = rows, dims[2] = experts."""
    dims: list[int]
    kind: int
    offset: int = 0
    shard: int = 0
    stride: int = 0
    bytes: int = 0

    @staticmethod
    def of(dims: list[int], kind: int) -> "Tensor":
        block, size = geometry(kind)
        if not dims or 0 in dims or dims[0] % block:
            raise InvalidData("invalid shape/alignment")
        stride = dims[0] // block * size
        total = stride
        for d in dims[1:]:
            total *= d
        return Tensor(list(dims), kind, 0, 0, stride, total)


@dataclass
class Matrix:
    """Host bytes of `count` stacked experts of rows x stride."""
    data: bytes | np.ndarray
    cols: int
    rows: int
    count: int
    kind: int
    stride: int

    @staticmethod
    def of(data, cols: int, rows: int, kind: int, count: int = 1) -> "Matrix":
        return Matrix(data, cols, rows, count, kind, stride_of(kind, cols))


class Buffer:
    """A device allocation or a view into one (the reference's Rc<Allocation> view)."""

    def __init__(self, gpu: "Gpu", ptr: int, nbytes: int, owner: "Buffer | None" = None):
        self.gpu, self.ptr, self.nbytes, self._owner = gpu, ptr, nbytes, owner
        self._owned = owner is None
        self._pooled = False          # an output buffer: goes back to the handle's size-keyed pool

    def view_f32(self, offset: int, count: int) -> "Buffer":
        if offset < 0 or count < 0 or (offset + count) * 4 > self.nbytes:
            raise InvalidData("buffer view out of range")
        return Buffer(self.gpu, self.ptr + 4 * offset, 4 * count, self._owner or self)

    def view_bytes(self, offset: int, nbytes: int) -> "Buffer":
        if offset < 0 or nbytes < 0 or offset + nbytes > self.nbytes:
            raise InvalidData("buffer view out of range")
        return Buffer(self.gpu, self.ptr + offset, nbytes, self._owner or self)

    def release(self) -> None:
        if self._owned and self.ptr and self.gpu._h:
            if self._pooled:
                self.gpu._lib.ingot_output_release(self.gpu._h, self.ptr)
            else:
                self.gpu._lib.ingot_buffer_free(self.gpu._h, self.ptr)
        self.ptr = 0

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class Command:
    """Work issued between command() and finish()/complete(); optionally recorded."""

    def __init__(self, gpu: "Gpu"):
        self.gpu = gpu


class Graph:
    """A recorded command that can be replayed (one decode step in one submission)."""

    def __init__(self, gpu: "Gpu", handle: int):
        self.gpu, self._g = gpu, handle

    def submit(self) -> None:
        self.gpu._check(self.gpu._lib.ingot_command_submit(self.gpu._h, self._g))

    def __del__(self):
        try:
            if self._g:
                self.gpu._lib.ingot_command_destroy(self._g)
                self._g = 0
        except Exception:
            pass


class _HostMatrix(C.Structure):
    _fields_ = [("data", C.c_void_p), ("bytes", C.c_size_t), ("cols", C.c_uint64), ("rows", C.c_uint64), ("count", C.c_uint64),
                ("kind", C.c_uint32), ("stride", C.c_uint64)]


class _RopeParams(C.Structure):
    _fields_ = [("head_dim", C.c_uint32), ("heads", C.c_uint32), ("kv_heads", C.c_uint32), ("rotated", C.c_uint32),
                ("position", C.c_uint32), ("base", C.c_float), ("neox", C.c_uint32), ("use_factors", C.c_uint32),
                ("qk_norm", C.c_uint32), ("eps", C.c_float), ("value_norm", C.c_uint32), ("q_scale", C.c_float)]


class _EpBuffers(C.Structure):
    _fields_ = [("rx_rows", C.c_void_p), ("rx_meta", C.c_void_p), ("rx_ready", C.c_void_p), ("ret_rows", C.c_void_p),
                ("ret_ready", C.c_void_p)]


class EpExchange:
    """The areas of one rank's window that the expert-parallel token exchange uses (ingot_ep_*): `cap` places
    per sending rank, rows of `hidden` floats."""

    def __init__(self, group: "Group", cap: int, hidden: int):
        self.group, self.cap, self.hidden = group, cap, hidden
        w = group.world
        self.rx_rows = group.alloc(w * cap * hidden)
        self.rx_meta = group.alloc(w * cap)
        self.rx_ready = group.alloc(2 * w)
        self.ret_rows = group.alloc(cap * hidden)
        self.ret_ready = group.alloc(2 * w)
        self._c = _EpBuffers(self.rx_rows.ptr, self.rx_meta.ptr, self.rx_ready.ptr, self.ret_rows.ptr, self.ret_ready.ptr)

    @staticmethod
    def window_bytes(world: int, cap: int, hidden: int) -> int:
        return 4 * (world * cap * hidden + world * cap + 4 * world + cap * hidden) + 5 * 256

    def dispatch(self, slot: int, x: "Buffer", ids: "Buffer", tokens: int, top: int, experts_per_rank: int) -> None:
        g = self.group.gpu
        g._check(g._lib.ingot_ep_dispatch(self.group._g, slot, C.byref(self._c), x.ptr, ids.ptr, tokens, top, self.hidden, self.cap,
                                          experts_per_rank))

    def receive(self, slot: int, ids_out: "Buffer") -> None:
        g = self.group.gpu
        g._check(g._lib.ingot_ep_receive(self.group._g, slot, C.byref(self._c), self.hidden, self.cap, ids_out.ptr))

    def give_back(self, slot: int, rows: "Buffer", inverse: "Buffer | None" = None) -> None:
        g = self.group.gpu
        g._check(g._lib.ingot_ep_return(self.group._g, slot, C.byref(self._c), rows.ptr, inverse.ptr if inverse else None, self.hidden,
                                        self.cap))

    def combine(self, slot: int, weights: "Buffer", top: int, tokens: int, y: "Buffer") -> None:
        g = self.group.gpu
        g._check(g._lib.ingot_ep_combine(self.group._g, slot, C.byref(self._c), weights.ptr, self.hidden, top, tokens, self.cap, y.ptr))


class Group:
    """One rank's end of a tensor-parallel group (ingot_group_*): a window of device memory the other ranks
    write into, and the exchange slots the projections signal and wait for."""
    NO_SLOT = 0xFFFFFFFF

    def __init__(self, gpu: "Gpu", rank: int, world: int, window_bytes: int, slots: int):
        self.gpu, self.rank, self.world, self.window_bytes = gpu, rank, world, window_bytes
        h, handle = C.c_void_p(), (C.c_uint8 * 64)()
        gpu._check(gpu._lib.ingot_group_create(gpu._h, rank, world, window_bytes, slots, C.byref(h), handle))
        self._g, self.handle, self._used = h.value, bytes(handle), 0

    def connect(self, handles: bytes) -> None:
        """`handles`: the 64-byte handles of all ranks, in rank order (one process per GPU)."""
        buf = (C.c_uint8 * len(handles)).from_buffer_copy(handles)
        self.gpu._check(self.gpu._lib.ingot_group_connect(self._g, buf))

    @staticmethod
    def connect_local(groups: "list[Group]") -> None:
        """All ranks live in this process (one handle per device)."""
        arr = (C.c_void_p * len(groups))(*[g._g for g in groups])
        st = groups[0].gpu._lib.ingot_group_connect_local(arr, len(groups))
        if st != _abi.OK:
            raise DeviceError("cannot connect the group's windows (peer access between the devices)")

    def window(self, rank: int | None = None) -> int:
        p = C.c_void_p()
        self.gpu._check(self.gpu._lib.ingot_group_window(self._g, self.rank if rank is None else rank, C.byref(p)))
        return p.value

    def alloc(self, n_f32: int) -> "Buffer":
        """float32 vector inside the own window; every rank allocates in the same order, so offsets agree."""
        off = (self._used + 255) & ~255
        if off + 4 * n_f32 > self.window_bytes:
            raise InvalidData("group window exhausted")
        self._used = off + 4 * n_f32
        holder = Buffer(self.gpu, 0, 0)
        return Buffer(self.gpu, self.window() + off, 4 * n_f32, holder)       # a view: the window owns the memory

    def step(self) -> None:
        self.gpu._check(self.gpu._lib.ingot_group_step(self._g))

    def wait(self, slot: int, whole: "Buffer") -> None:
        """Enqueues the collection of every rank's rows of `slot` in this step into the plain vector `whole`."""
        self.gpu._check(self.gpu._lib.ingot_group_wait(self._g, slot, whole.ptr, whole.nbytes // 4))

    def signal_next(self, slot: int) -> None:
        self.gpu._check(self.gpu._lib.ingot_tp_signal_next(self._g, slot))

    def wait_next(self, slot_a: int, slot_b: int | None = None) -> None:
        self.gpu._check(self.gpu._lib.ingot_tp_wait_next(self._g, slot_a, self.NO_SLOT if slot_b is None else slot_b))

    def close(self) -> None:
        if self._g:
            self.gpu._lib.ingot_group_destroy(self._g)
            self._g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Chain:
    """A recorded sequence of fused-norm projections that runs as one persistent kernel."""

    def __init__(self, gpu: "Gpu", handle: int):
        self.gpu, self._c = gpu, handle

    def submit(self) -> None:
        self.gpu._check(self.gpu._lib.ingot_chain_submit(self.gpu._h, self._c))

    def info(self) -> dict:
        v = [C.c_uint32() for _ in range(4)]
        self.gpu._check(self.gpu._lib.ingot_chain_info(self._c, *[C.byref(x) for x in v]))
        return dict(zip(("projections", "waits", "stages", "stage_bytes"), (x.value for x in v)))

    def __del__(self):
        try:
            if self._c:
                self.gpu._lib.ingot_chain_destroy(self._c)
                self._c = 0
        except Exception:
            pass


@dataclass
class Weight:
    """A device buffer plus its tensor descriptor (src/weights.rs:10-13)."""
    buffer: Buffer
    t: Tensor

    def require_f32(self) -> None:
        if self.t.kind != F32:
            raise InvalidData("normalization/state parameters require F32 weights")

    @staticmethod
    def load(gpu: "Gpu", data, shape: list[int], kind: int, expect: list[int] | None = None) -> "Weight":
        t = Tensor.of(shape, kind)
        if expect is not None and list(expect) != list(shape):
            raise InvalidData(f"expected {expect}, found {shape}")
        return Weight(gpu.load_weight(data, t), t)

    def project(self, gpu: "Gpu", c: Command, x: Buffer) -> Buffer:
        rows = self.t.dims[1] if len(self.t.dims) > 1 else 1
        return gpu.matvec(c, self.buffer, self.t.dims[0], rows, self.t.stride, self.t.kind, x)


def _as_u8(data) -> np.ndarray:
    if isinstance(data, np.ndarray):
        return np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    return np.frombuffer(bytes(data), dtype=np.uint8)


class Gpu:
    """One CUDA device, one stream, one owner thread (the reference's Gpu)."""

    VECTOR_KINDS = (Q4_K, Q6_K, Q4_0, Q8_0, F16, F32, BF16)

    def __init__(self, device: int = 0):
        self._lib = _abi.load()
        h = C.c_void_p()
        st = self._lib.ingot_gpu_create(device, C.byref(h))
        if st != _abi.OK:
            raise DeviceError(f"cannot create a B200 (sm_100) handle on CUDA device {device}")
        self._h = h.value

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ingot_gpu_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- errors ----
    def _check(self, status: int) -> None:
        if status == _abi.OK:
            return
        msg = (self._lib.ingot_last_error(self._h) or b"").decode()
        if status in (_abi.INVALID, _abi.UNSUPPORTED, _abi.EOF):
            raise InvalidData(msg)
        if status == _abi.TIMEOUT:
            raise DeviceTimeout(msg)
        raise DeviceError(msg)

    def set_option(self, option: int, value: int) -> None:
        self._check(self._lib.ingot_gpu_set_option(self._h, option, value))

    def set_stream(self, cuda_stream: int | None) -> None:
        self._check(self._lib.ingot_gpu_set_stream(self._h, cuda_stream))

    # ---- buffers ----
    def empty_bytes(self, n: int) -> Buffer:
        p = C.c_void_p()
        self._check(self._lib.ingot_buffer_alloc(self._h, n, C.byref(p)))
        return Buffer(self, p.value, n)

    def bytes(self, data) -> Buffer:
        raw = _as_u8(data)
        b = self.empty_bytes(raw.size)
        self._check(self._lib.ingot_buffer_upload(self._h, b.ptr, raw.ctypes.data, raw.size))
        self._check(self._lib.ingot_synchronize(self._h))
        return b

    def floats(self, values) -> Buffer:
        return self.bytes(np.ascontiguousarray(values, dtype=np.float32))

    def bf16(self, values) -> Buffer:
        """Uploads float32 values rounded to bfloat16."""
        from .synth import to_bf16_bits
        return self.bytes(to_bf16_bits(np.ascontiguousarray(values, dtype=np.float32)))

    def zeros(self, n_f32: int) -> Buffer:
        b = self.empty_bytes(4 * n_f32)
        self._check(self._lib.ingot_buffer_zero(self._h, b.ptr, 4 * n_f32))
        return b

    def output(self, n_f32: int) -> Buffer:
        """Gpu::output (src/metal.rs:1278-1333): a float32 buffer from the size-keyed pool (a plain allocation while
        no workspace budget is set)."""
        p = C.c_void_p()
        self._check(self._lib.ingot_output_alloc(self._h, n_f32, C.byref(p)))
        b = Buffer(self, p.value, 4 * n_f32)
        b._pooled = True
        return b

    def configure_workspace(self, limit: int) -> None:
        """Gpu::configure_workspace (src/metal.rs:1335-1337)."""
        self._check(self._lib.ingot_gpu_configure_workspace(self._h, limit))

    def workspace_statistics(self) -> tuple[int, int, int, int]:
        """Cumulative new allocations, reuse count, current managed bytes and peak bytes (src/metal.rs:1338-1342)."""
        a, r, m, pk = C.c_uint64(), C.c_uint64(), C.c_size_t(), C.c_size_t()
        self._check(self._lib.ingot_workspace_statistics(self._h, C.byref(a), C.byref(r), C.byref(m), C.byref(pk)))
        return a.value, r.value, m.value, pk.value

    def load_weight(self, data, t: Tensor) -> Buffer:
        raw = _as_u8(data)
        p = C.c_void_p()
        dims = list(t.dims) + [1] * (3 - len(t.dims))
        count = 1
        for d in dims[2:]:
            count *= d
        self._check(self._lib.ingot_weight_upload(self._h, raw.ctypes.data, t.kind, dims[0], dims[1], count,
                                                  raw.size, C.byref(p)))
        self._check(self._lib.ingot_synchronize(self._h))
        return Buffer(self, p.value, raw.size)

    # ---- commands ----
    def command(self) -> Command:
        return Command(self)

    def record(self) -> None:
        self._check(self._lib.ingot_command_begin(self._h))

    def end_record(self) -> Graph:
        g = C.c_void_p()
        self._check(self._lib.ingot_command_end(self._h, C.byref(g)))
        return Graph(self, g.value)

    def chain_begin(self) -> None:
        self._check(self._lib.ingot_chain_begin(self._h))

    def chain_end(self) -> Chain:
        c = C.c_void_p()
        self._check(self._lib.ingot_chain_end(self._h, C.byref(c)))
        return Chain(self, c.value)

    def complete(self, cmd: Command | None = None) -> None:
        self._check(self._lib.ingot_synchronize(self._h))

    def read_bytes(self, b: Buffer, n: int | None = None) -> np.ndarray:
        n = b.nbytes if n is None else n
        out = np.empty(n, dtype=np.uint8)
        self._check(self._lib.ingot_buffer_read(self._h, out.ctypes.data, b.ptr, n))
        return out

    def read_f32(self, b: Buffer, n: int | None = None) -> np.ndarray:
        n = b.nbytes // 4 if n is None else n
        return self.read_bytes(b, 4 * n).view(np.float32)

    def read_u32(self, b: Buffer, n: int) -> np.ndarray:
        return self.read_bytes(b, 4 * n).view(np.uint32)

    def finish(self, cmd: Command, out: Buffer) -> np.ndarray:
        """Waits, checks the device status and returns `out`; rejects non-finite values."""
        self.complete(cmd)
        values = self.read_f32(out)
        if not np.isfinite(values).all():
            raise InvalidData("output contains non-finite values")
        return values

    # ---- operators on buffers ----
    @staticmethod
    def _xk(x_kind: int) -> int:
        return x_kind

    def matvec(self, cmd, w: Buffer, cols, rows, stride, kind, x: Buffer, x_kind: int = F32) -> Buffer:
        return self.matmul(cmd, w, cols, rows, stride, kind, 0, x, 1, x_kind)

    def matmul(self, cmd, w: Buffer, cols, rows, stride, kind, expert, x: Buffer, count, x_kind: int = F32,
               out: Buffer | None = None) -> Buffer:
        y = out or self.output(rows * count)
        self._check(self._lib.ingot_matmul(self._h, w.ptr, cols, rows, stride, kind, expert, x.ptr, x_kind, count,
                                           y.ptr))
        return y

    def gemm(self, cmd, w: Buffer, cols, rows, stride, kind, expert, x: Buffer, count, x_kind: int = F32,
             out: Buffer | None = None) -> Buffer:
        """The tensor-core prefill GEMM (the reference's gemm_q4k / gemm_q6k)."""
        y = out or self.output(rows * count)
        self._check(self._lib.ingot_gemm(self._h, w.ptr, cols, rows, stride, kind, expert, x.ptr, x_kind, count, y.ptr))
        return y

    def generic_project(self, cmd, w: Weight, x: Buffer, count: int, x_kind: int = F32):
        if w.t.kind not in self.VECTOR_KINDS:
            return None
        return self.matmul(cmd, w.buffer, w.t.dims[0], w.t.dims[1], w.t.stride, w.t.kind, 0, x, count, x_kind)

    def generic_gate_up(self, cmd, gate_up, x: Buffer, count: int, gelu: bool, x_kind: int = F32):
        gate, up = gate_up
        same = gate.t.kind == up.t.kind and gate.t.stride == up.t.stride and gate.t.dims == up.t.dims
        if not same or gate.t.kind not in self.VECTOR_KINDS:
            return None
        rows = gate.t.dims[1]
        y = self.output(rows * count)
        self._check(self._lib.ingot_gate_up(self._h, gate.buffer.ptr, up.buffer.ptr, gate.t.dims[0], rows,
                                            gate.t.stride, gate.t.kind, x.ptr, x_kind, count, int(gelu), y.ptr))
        return y

    def generic_routed_gate_up(self, cmd, gate_up, x_ids, top: int, pairs: int, x_kind: int = F32):
        gate, up = gate_up
        x, ids = x_ids
        same = gate.t.kind == up.t.kind and gate.t.stride == up.t.stride and gate.t.dims == up.t.dims
        if not same or gate.t.kind not in self.VECTOR_KINDS:
            return None
        t = gate.t
        experts = t.dims[2] if len(t.dims) > 2 else 1
        y = self.output(t.dims[1] * pairs)
        self._check(self._lib.ingot_routed_gate_up(self._h, gate.buffer.ptr, up.buffer.ptr, t.dims[0], t.dims[1],
                                                   t.stride, t.kind, experts, x.ptr, x_kind, ids.ptr, top, pairs,
                                                   y.ptr))
        return y

    def generic_routed(self, cmd, w: Weight, x_ids_y, per_pair: bool, top: int, pairs: int,
                       x_kind: int = F32) -> bool:
        x, ids, y = x_ids_y
        if w.t.kind not in self.VECTOR_KINDS:
            return False
        experts = w.t.dims[2] if len(w.t.dims) > 2 else 1
        self._check(self._lib.ingot_routed(self._h, w.buffer.ptr, w.t.dims[0], w.t.dims[1], w.t.stride, w.t.kind,
                                           experts, x.ptr, x_kind, ids.ptr, int(per_pair), top, pairs, y.ptr))
        return True

    def activation(self, cmd, gate: Buffer, up: Buffer, count: int, gelu: bool = False) -> Buffer:
        y = self.output(count)
        self._check(self._lib.ingot_activation(self._h, gate.ptr, up.ptr, count, int(gelu), y.ptr))
        return y

    def merge(self, cmd, routed: Buffer, shared: Buffer, weights: Buffer, shared_logit: Buffer, width: int,
              top: int) -> Buffer:
        y = self.output(width)
        self._check(self._lib.ingot_merge(self._h, routed.ptr, shared.ptr, weights.ptr, shared_logit.ptr, width,
                                          top, y.ptr))
        return y

    def add_rms(self, cmd, a: Buffer, b: Buffer | None, w: Buffer | None, width: int, rows: int, eps: float,
                add: bool = True, bf16_out: bool = False):
        """(s, y[, y_bf16]) like the reference's add_rms (src/metal_generic.rs:94-125)."""
        s = self.output(width * rows) if add else None
        y = self.output(width * rows)
        yb = self.empty_bytes(2 * width * rows) if bf16_out else None
        self._check(self._lib.ingot_add_rms(self._h, a.ptr, b.ptr if b else None, w.ptr if w else None,
                                            s.ptr if s else None, y.ptr, yb.ptr if yb else None, width, rows,
                                            float(eps), int(add)))
        return (s, y, yb) if bf16_out else (s, y)

    def op(self, cmd, name: str, buffers, params, width: int = 1, height: int = 1) -> None:
        """String-dispatched launcher for the reference's `Gpu::op` call sites on this
        path (src/metal.rs:686); `params` are the kernel's p[] words."""
        p = [int(v) for v in params]
        b = buffers
        if name == "read_rows":               # p: cols, rows, stride, kind
            self._check(self._lib.ingot_dequant_rows(self._h, b[0].ptr, p[0], p[1], p[2], p[3], b[1].ptr))
        elif name in ("route_topk", "route_gpu", "route_gpu_batch"):   # p: experts, top ; height/width tokens
            tokens = max(width, height) if name != "route_gpu" else 1
            self._check(self._lib.ingot_route_topk(self._h, b[0].ptr, p[0], p[1], tokens, b[1].ptr, b[2].ptr))
        elif name == "moe_sum":               # p: width, top, tokens
            self._check(self._lib.ingot_moe_sum(self._h, b[0].ptr, b[1].ptr, p[0], p[1], p[2], b[2].ptr))
        elif name == "project_routed_batch":  # p: cols, rows, stride, kind, top, per_pair ; height = pairs
            experts = b[0].nbytes // (p[1] * p[2])
            self._check(self._lib.ingot_routed(self._h, b[0].ptr, p[0], p[1], p[2], p[3], experts, b[1].ptr, F32,
                                               b[2].ptr, p[5], p[4], height, b[3].ptr))
        else:
            raise InvalidData(f"no operator named {name} on this path")

    def independent(self):
        """Scope in which only operators that do not consume each other's results are issued; they run
        concurrently (Gpu::independent_projections, src/metal.rs:1371-1396)."""
        gpu = self

        class _Scope:
            def __enter__(self_inner):
                gpu._check(gpu._lib.ingot_independent_begin(gpu._h))

            def __exit__(self_inner, *exc):
                gpu._check(gpu._lib.ingot_independent_end(gpu._h))
                return False

        return _Scope()

    def packed_x_bytes(self, cols: int) -> int:
        n = C.c_uint64()
        self._check(self._lib.ingot_packed_x_bytes(cols, C.byref(n)))
        return n.value

    def pack_x(self, x: Buffer, rows: int, cols: int, x_kind: int = F32, out: Buffer | None = None) -> Buffer:
        """Packs activation rows for the tensor-core GEMV; pass the result with x_kind=X_PACKED."""
        p = out or self.empty_bytes(rows * self.packed_x_bytes(cols))
        self._check(self._lib.ingot_pack_x(self._h, x.ptr, x_kind, rows, cols, p.ptr))
        return p

    def packed_hi_bytes(self, cols: int) -> int:
        n = C.c_uint64()
        self._check(self._lib.ingot_packed_hi_bytes(cols, C.byref(n)))
        return n.value

    def pack_x_hi(self, x_bf16: Buffer, rows: int, cols: int, out: Buffer | None = None) -> Buffer:
        """Packs bfloat16 activation rows as high-part rows; pass the result with x_kind=X_PACKED_HI."""
        p = out or self.empty_bytes(rows * self.packed_hi_bytes(cols))
        self._check(self._lib.ingot_pack_x_hi(self._h, x_bf16.ptr, rows, cols, p.ptr))
        return p

    def packed_digits_bytes(self, cols: int) -> int:
        n = C.c_uint64()
        self._check(self._lib.ingot_packed_digits_bytes(cols, C.byref(n)))
        return n.value

    def pack_digits(self, x: Buffer, rows: int, cols: int, x_kind: int = F32, out: Buffer | None = None) -> Buffer:
        """Packs activation rows as base-256 digits for the tcgen05 int8 GEMV; pass the result with x_kind=X_DIGITS."""
        p = out or self.empty_bytes(rows * self.packed_digits_bytes(cols))
        self._check(self._lib.ingot_pack_digits(self._h, x.ptr, x_kind, rows, cols, p.ptr))
        return p

    # ---- the rest of a generic decode step ----
    def embedding_batch(self, cmd, w: Weight, ids: Buffer, count: int) -> Buffer:
        """Rows ids[t] of the embedding matrix as float32 (embedding_batch, kernels/qwen.metal:139)."""
        t = w.t
        y = self.output(t.dims[0] * count)
        self._check(self._lib.ingot_embedding_batch(self._h, w.buffer.ptr, ids.ptr, t.dims[0], t.dims[1], t.stride, t.kind, count, y.ptr))
        return y

    def qk_rope_cache(self, cmd, q: Buffer, k: Buffer, v: Buffer, q_out: Buffer, k_cache: Buffer, v_cache: Buffer, *, head_dim: int,
                      heads: int, kv_heads: int, rotated: int, position: int, base: float, tokens: int, neox: bool = False,
                      factors: Buffer | None = None, q_norm: Buffer | None = None, k_norm: Buffer | None = None, eps: float = 1e-6,
                      value_norm: bool = False, q_scale: float = 1.0) -> None:
        """qk_rope_cache (kernels/generic.metal:405-438)."""
        p = _RopeParams(head_dim, heads, kv_heads, rotated, position, base, int(neox), int(factors is not None),
                        int(q_norm is not None), eps, int(value_norm), q_scale)
        ptr = lambda b: b.ptr if b is not None else None
        self._check(self._lib.ingot_qk_rope_cache(self._h, q.ptr, k.ptr, v.ptr, ptr(q_norm), ptr(k_norm), ptr(factors), q_out.ptr,
                                                  k_cache.ptr, v_cache.ptr, C.byref(p), tokens))

    def attention_decode(self, cmd, q: Buffer, k_cache: Buffer, v_cache: Buffer, head_dim: int, heads: int, kv_heads: int,
                         position: int, tokens: int, window: int = 0):
        """attention_decode_<D> (kernels/generic.metal:440-474); None when there is no kernel for the head dimension."""
        out = self.output(tokens * heads * head_dim)
        st = self._lib.ingot_attention_decode(self._h, q.ptr, k_cache.ptr, v_cache.ptr, out.ptr, head_dim, heads, kv_heads, position,
                                              window, tokens)
        if st == _abi.UNSUPPORTED:
            return None
        self._check(st)
        return out

    # ---- architecture glue of the generic path (kernels/generic_arch.metal:2-17) ----
    def scale_rows(self, cmd, x: Buffer, n: int, scale: float) -> Buffer:
        y = self.output(n)
        self._check(self._lib.ingot_scale_rows(self._h, x.ptr, n, scale, y.ptr))
        return y

    def softcap_rows(self, cmd, x: Buffer, n: int, cap: float) -> Buffer:
        y = self.output(n)
        self._check(self._lib.ingot_softcap_rows(self._h, x.ptr, n, cap, y.ptr))
        return y

    def swiglu_fused(self, cmd, x: Buffer, tokens: int, ff: int) -> Buffer:
        y = self.output(tokens * ff)
        self._check(self._lib.ingot_swiglu_fused(self._h, x.ptr, tokens, ff, y.ptr))
        return y

    def copy_columns(self, cmd, x: Buffer, rows: int, width: int, offset: int, stride: int) -> Buffer:
        y = self.output(rows * width)
        self._check(self._lib.ingot_copy_columns(self._h, x.ptr, rows, width, offset, stride, y.ptr))
        return y

    def attention_prefill(self, cmd, q: Buffer, k_cache: Buffer, v_cache: Buffer, head_dim: int, heads: int, kv_heads: int,
                          position: int, rows: int, window: int = 0):
        """Generic::flash (src/generic.rs:421-470; flash_prefill_<D>, kernels/generic.metal:19-136): causal attention of
        `rows` query rows from `position` on; None when there is no kernel for the head dimension."""
        out = self.output(rows * heads * head_dim)
        st = self._lib.ingot_attention_prefill(self._h, q.ptr, k_cache.ptr, v_cache.ptr, out.ptr, head_dim, heads, kv_heads,
                                               position + rows, position, rows, window)
        if st == _abi.UNSUPPORTED:
            return None
        self._check(st)
        return out

    def finish_greedy(self, cmd, logits: Buffer, rows: int, vocabulary: int, mapping: Buffer | None = None) -> list[int]:
        """Gpu::finish_greedy (src/metal.rs:1507-1548): the greedy token of every row; non-finite logits are an error."""
        chunks = (vocabulary + 1023) // 1024
        partial, result = self.empty_bytes(4 * rows * chunks * 3), self.empty_bytes(4 * rows * 2)
        self._check(self._lib.ingot_greedy_select(self._h, logits.ptr, mapping.ptr if mapping else None, rows, vocabulary, partial.ptr,
                                                  result.ptr))
        self.complete(cmd)
        out = self.read_u32(result, rows * 2).reshape(rows, 2)
        if out[:, 1].any():
            raise InvalidData("non-finite logits")
        return [int(v) for v in out[:, 0]]

    def route_topk(self, logits: Buffer, experts: int, top: int, tokens: int):
        ids = self.empty_bytes(4 * top * tokens)
        w = self.output(top * tokens)
        self._check(self._lib.ingot_route_topk(self._h, logits.ptr, experts, top, tokens, ids.ptr, w.ptr))
        return ids, w

    def moe_sum(self, routed: Buffer, weights: Buffer, width: int, top: int, tokens: int) -> Buffer:
        y = self.output(width * tokens)
        self._check(self._lib.ingot_moe_sum(self._h, routed.ptr, weights.ptr, width, top, tokens, y.ptr))
        return y

    def expert_layout(self, ids: Buffer, pairs: int, experts: int, tile_capacity: int):
        layout = self.empty_bytes(8 * experts)
        tiles = self.empty_bytes(16 * max(tile_capacity, 1))
        packed = self.empty_bytes(4 * max(pairs, 1))
        inverse = self.empty_bytes(4 * max(pairs, 1))
        self._check(self._lib.ingot_expert_layout(self._h, ids.ptr, pairs, experts, tile_capacity, layout.ptr,
                                                  tiles.ptr, packed.ptr, inverse.ptr))
        return layout, tiles, packed, inverse

    def combine_packed(self, routed: Buffer, weights: Buffer, inverse: Buffer, width: int, top: int,
                       tokens: int) -> Buffer:
        y = self.output(width * tokens)
        self._check(self._lib.ingot_combine_packed(self._h, routed.ptr, weights.ptr, inverse.ptr, width, top,
                                                   tokens, y.ptr))
        return y

    # ---- host-vector conveniences (the reference's public parity hooks) ----
    def dequant(self, m: Matrix) -> np.ndarray:
        raw = _as_u8(m.data)
        out = np.empty(max(m.cols * m.rows * m.count, 1), dtype=np.float32)
        self._check(self._lib.ingot_dequant_host(self._h, raw.ctypes.data, raw.size, m.cols, m.rows, m.count,
                                                 m.kind, m.stride, out.ctypes.data))
        return out[: m.cols * m.rows * m.count]

    def ffn(self, matrices, x: Buffer) -> Buffer:
        """Gpu::ffn (src/metal.rs:1634-1661): every stacked expert's SwiGLU FFN of the same input;
        returns `count` rows of `down.rows` values (ingot_ffn on device buffers)."""
        gate, up, down = matrices
        if (gate.cols, gate.rows, gate.count, gate.kind) != (up.cols, up.rows, up.count, up.kind) or \
                (down.cols, down.rows, down.count, down.kind) != (gate.rows, gate.cols, gate.count, gate.kind):
            raise InvalidData("FFN matrix shapes do not match")
        bufs = [self.bytes(_as_u8(m.data)) for m in matrices]
        scratch = self.empty_bytes(4 * 3 * gate.rows * gate.count)
        ids = self.bytes(np.arange(gate.count, dtype=np.uint32).view(np.uint8))
        out = self.output(down.rows * down.count)
        self._check(self._lib.ingot_ffn(self._h, bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, gate.cols, gate.rows, gate.count, gate.kind,
                                        x.ptr, scratch.ptr, ids.ptr, out.ptr))
        self._check(self._lib.ingot_synchronize(self._h))          # the temporaries above are released on return
        return out

    def moe(self, routed, shared, shared_gate: Matrix, x, weights) -> np.ndarray:
        """Gpu::moe (src/metal.rs:1663-1713): the FFNs of the selected experts (stacked in `routed`, one
        weight each) and of the shared expert, merged as sum_e w_e * routed_e + sigmoid(shared_gate . x) * shared
        (ingot_moe_host does the checks and the work)."""
        xv = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        wv = np.ascontiguousarray(weights, dtype=np.float32).reshape(-1)
        keep = []

        def host(m: Matrix) -> _HostMatrix:
            raw = _as_u8(m.data)
            keep.append(raw)
            return _HostMatrix(raw.ctypes.data, raw.size, m.cols, m.rows, m.count, m.kind, m.stride)

        r3 = (_HostMatrix * 3)(*[host(m) for m in routed])
        s3 = (_HostMatrix * 3)(*[host(m) for m in shared])
        sg = host(shared_gate)
        out = np.empty(max(xv.size, 1), dtype=np.float32)
        self._check(self._lib.ingot_moe_host(self._h, r3, s3, C.byref(sg), xv.ctypes.data, xv.size, wv.ctypes.data, wv.size,
                                             out.ctypes.data))
        return out[:xv.size]

    def _validate(self, m: Matrix) -> None:
        """validate_matrix (src/metal.rs:1602-1621) through the library's own layout check."""
        raw = _as_u8(m.data)
        stride, total = C.c_uint64(), C.c_uint64()
        st = self._lib.ingot_tensor_layout(m.kind, m.cols, m.rows, m.count, C.byref(stride), C.byref(total))
        if st != _abi.OK or stride.value != m.stride or total.value != raw.size:
            raise InvalidData("matrix layout does not match its data")

    def project(self, m: Matrix, x) -> np.ndarray:
        raw = _as_u8(m.data)
        xv = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        out = np.empty(max(m.rows, 1), dtype=np.float32)
        self._check(self._lib.ingot_project_host(self._h, raw.ctypes.data, raw.size, m.cols, m.rows, m.count,
                                                 m.kind, m.stride, xv.ctypes.data, xv.size, out.ctypes.data))
        return out[: m.rows]
