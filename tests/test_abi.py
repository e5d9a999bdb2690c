"""CPU: the shared library loads, exports every symbol the header declares, and fails
loudly (no fallback) when there is no GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "train_station_b200.h")


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    src = re.sub(r"//[^\n]*", "", src)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}]*\)\s*;", src)
    return sorted(set(n for n in names if n not in ("defined",)))


def test_header_declares_the_reference_fifteen():
    ref = {"cuda_ffi_initialize", "cuda_ffi_cleanup", "get_cuda_device_count", "set_cuda_device",
           "get_current_cuda_device", "cuda_malloc", "cuda_free", "cuda_memcpy", "create_cuda_stream",
           "destroy_cuda_stream", "launch_add_kernel", "launch_sub_kernel", "launch_mul_kernel",
           "launch_matmul_kernel"}  # cuda_wrapper.h:10-31 (14 functions; the Rust side counts 15 with both memcpy directions)
    assert ref <= set(declared_symbols())


def test_every_declared_symbol_is_exported_and_bound(ts):
    lib = ts._ffi.lib()
    syms = declared_symbols()
    assert len(syms) > 80
    for name in syms:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in ts._ffi.SIGNATURES, f"{name} has no ctypes signature"
    for name in ts._ffi.SIGNATURES:
        assert name in syms, f"{name} bound in Python but not declared in the header"


def test_no_torch_types_in_signatures():
    src = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)   # declarations only, comments stripped
    assert "torch" not in src.lower() and "at::" not in src and "std::" not in src


def test_library_does_not_link_torch_or_the_oracle():
    import subprocess
    out = subprocess.run(["ldd", os.path.join(ROOT, "train-station_b200", "libtrain_station_b200.so")],
                         capture_output=True, text=True).stdout
    # NCCL is bound with dlopen on first use of data parallelism, so that a process which also imports
    # PyTorch (which bundles its own libnccl.so.2) ends up with a single copy whichever is loaded first
    assert "torch" not in out and "oracle" not in out and "nccl" not in out


def test_fails_loudly_without_a_gpu(ts):
    if ts.cuda_is_available():
        pytest.skip("a GPU is present")
    assert ts.cuda_device_count() == 0
    with pytest.raises(ts.TrainStationError):
        ts.Tensor.zeros([2, 2])
    lib = ts._ffi.lib()
    assert lib.cuda_ffi_initialize() is False
    assert lib.cuda_malloc(16) is None
    assert len(ts._ffi.last_error()) > 0
    # null pointers are refused before anything is launched (cuda_wrapper.cpp:64,70,76,82)
    assert lib.launch_matmul_kernel(None, None, None, 2, 2, 2, None) is False


def test_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "train-station_b200")
    for fn in os.listdir(pkg):
        if fn.endswith(".py"):
            assert "oracle" not in open(os.path.join(pkg, fn)).read(), fn
    for fn in os.listdir(os.path.join(pkg, "csrc")):
        assert "oracle" not in open(os.path.join(pkg, "csrc", fn)).read().lower(), fn


def test_rust_binding_file_is_current_and_complete():
    """include/train_station_b200.rs is what include/make_rust_bindings.py makes of the header today, and its extern
    block names every declared function with the argument count the header gives (no Rust toolchain here: the file is
    source for the reference's side, checked as text)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_rust_bindings", os.path.join(ROOT, "include", "make_rust_bindings.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    text = gen.generate()
    with open(os.path.join(ROOT, "include", "train_station_b200.rs")) as f:
        assert f.read() == text, "run python include/make_rust_bindings.py"
    bound = dict(re.findall(r"pub fn ([a-z_0-9]+)\((.*?)\)", text))
    assert sorted(bound) == declared_symbols()
    # the reference's own fifteen keep the spellings of src/cuda/mod.rs:139-208
    assert bound["cuda_malloc"] == "size: u64" and bound["cuda_memcpy"] == "dst: *mut f32, src: *const f32, size: u64, kind: i32"
    assert bound["launch_matmul_kernel"] == "a: *const f32, b: *const f32, result: *mut f32, m: u64, n: u64, k: u64, stream: *mut c_void"
    assert gen.rust_type("const float* const*") == "*const *const f32" and gen.rust_type("ts_tensor* const*") == "*const *mut TsTensor"
