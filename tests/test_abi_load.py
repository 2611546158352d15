"""The C-ABI library builds, loads and exports every symbol the header declares.
No compute calls: there is no GPU where this file runs."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT
from ingot_b200 import _abi, build


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _abi.load()


def header_names():
    text = open(os.path.join(ROOT, "include", "ingot_cuda.h")).read()
    return sorted(set(re.findall(r"INGOT_API\s+[\w\s\*]+?\b(ingot_\w+)\s*\(", text)))


def test_header_and_bindings_agree(lib):
    names = header_names()
    assert len(names) >= 30
    assert names == _abi.exported_names()
    for n in names:
        assert hasattr(lib, n), n


def test_only_the_abi_is_exported():
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", _abi.LIB_PATH], capture_output=True, text=True).stdout
    syms = [l.split()[-1] for l in out.splitlines() if " T " in l]
    assert syms and all(s.startswith("ingot_") for s in syms), [s for s in syms if not s.startswith("ingot_")][:5]


def test_geometry_and_layout_need_no_gpu(lib):
    b, s = C.c_uint32(), C.c_uint32()
    assert lib.ingot_geometry(12, C.byref(b), C.byref(s)) == _abi.OK and (b.value, s.value) == (256, 144)
    assert lib.ingot_geometry(14, C.byref(b), C.byref(s)) == _abi.OK and (b.value, s.value) == (256, 210)
    assert lib.ingot_geometry(13, C.byref(b), C.byref(s)) == _abi.UNSUPPORTED
    st, by = C.c_uint64(), C.c_uint64()
    assert lib.ingot_tensor_layout(14, 4096, 151936, 1, C.byref(st), C.byref(by)) == _abi.OK
    assert (st.value, by.value) == (3360, 510504960)
    assert lib.ingot_tensor_layout(12, 2048, 768, 128, C.byref(st), C.byref(by)) == _abi.OK and by.value == 128 * 884736
    assert lib.ingot_tensor_layout(12, 100, 1, 1, C.byref(st), C.byref(by)) == _abi.INVALID
    assert lib.ingot_tensor_layout(12, 1 << 40, 1 << 40, 1 << 20, C.byref(st), C.byref(by)) == _abi.INVALID


def test_no_device_is_a_loud_error(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.ingot_gpu_create(0, C.byref(h)) == _abi.DEVICE and not h.value
    from ingot_b200 import DeviceError, Gpu
    with pytest.raises(DeviceError):
        Gpu(0)


def test_missing_library_is_a_loud_error(monkeypatch):
    monkeypatch.setattr(_abi, "_lib", None)
    monkeypatch.setattr(_abi, "LIB_PATH", "/nonexistent/libingot_cuda.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _abi.load()


def test_rust_sys_bindings_name_every_declared_function():
    """include/rust/ingot-cuda-sys/src/lib.rs is generated from the header: regenerating it changes nothing, and
    it declares every INGOT_API function."""
    import importlib.util
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rs_path = os.path.join(root, "include", "rust", "ingot-cuda-sys", "src", "lib.rs")
    committed = open(rs_path).read()
    header = open(os.path.join(root, "include", "ingot_cuda.h")).read()
    header = re.sub(r"/\*.*?\*/", " ", header, flags=re.S)
    declared = set(re.findall(r"INGOT_API\s+[^;{]*?\b(ingot_\w+)\s*\(", header))
    bound = set(re.findall(r"pub fn (ingot_\w+)\(", committed))
    assert declared and declared == bound, sorted(declared ^ bound)
    spec = importlib.util.spec_from_file_location("gen_sys", os.path.join(root, "include", "rust", "gen_sys.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    gen.main()
    assert open(rs_path).read() == committed, "run python include/rust/gen_sys.py"
