"""CPU checks of the drop-in boundary: the shared library loads, exports every symbol that
include/nne_cuda.h declares, the ctypes table covers the header, and argument errors that need
no device come back as status codes.  No compute call is made here."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "nne_cuda.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"NNE_API\s+[\w\s\*]+?\b(nne_\w+)\s*\(", text)))


def test_header_declares_expected_surface():
    syms = declared_symbols()
    for must in ["nne_cuda_ctx_create", "nne_quantize_rows", "nne_quantize_tensor",
                 "nne_qlinear_create_from_f32", "nne_qlinear_create_from_i8",
                 "nne_qlinear_download", "nne_qlinear_forward_host", "nne_qlinear_forward_dev",
                 "nne_status_string", "nne_last_error"]:
        assert must in syms


def test_library_exports_every_declared_symbol(nne):
    lib = nne.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in nne_cuda.h but not exported"


def test_ctypes_table_matches_header(nne):
    from importlib import import_module
    table = import_module("neural-network-engine_b200._lib").SIGNATURES
    assert sorted(table) == declared_symbols()


def test_static_archive_is_built():
    assert os.path.exists(os.path.join(ROOT, "neural-network-engine_b200", "lib", "libnne_cuda.a"))


def test_status_strings_and_null_arguments(nne):
    lib = nne.load()
    assert lib.nne_status_string(0) == b"ok"
    assert lib.nne_status_string(2) == b"shape mismatch"
    assert lib.nne_status_string(99) == b"unknown status"
    # null handles are rejected before any device work
    assert lib.nne_qlinear_forward_host(None, None, 1, 1, None) == 1
    assert lib.nne_cuda_ctx_create(0, None) == 1
    buf = C.create_string_buffer(256)
    assert lib.nne_last_error(buf, 256) == 0 and b"null" in buf.value
    assert lib.nne_qlinear_destroy(None) == 0 and lib.nne_cuda_ctx_destroy(None) == 0
    assert lib.nne_qlinear_memory_bytes(None) == 0


def test_no_device_is_an_error_not_a_fallback(nne):
    """Without a usable sm_100 device context creation fails; nothing computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(nne.GpuError):
        nne.CudaContext(0)
    lin = nne.Linear([[1.0, 2.0], [3.0, 4.0]])
    ql = nne.QLinear.from_linear(lin)           # infallible, like the reference
    with pytest.raises(nne.GpuError):           # the stored failure surfaces at forward
        ql.forward([[1.0, 1.0]])


def test_host_side_validation_needs_no_device(nne):
    import numpy as np
    ql = nne.QLinear(np.zeros(6, np.int8), np.ones(3, np.float32), None, 2, 3)
    with pytest.raises(nne.InvalidArgument):    # reference :149-154
        ql.forward(np.zeros(2, np.float32))
    with pytest.raises(nne.ShapeMismatch) as e: # reference :156-162
        ql.forward(np.zeros((4, 5), np.float32))
    assert e.value.expected == [2] and e.value.actual == [5]
    assert ql.memory_bytes() == 6 + 12 and ql.parameters() == []


def test_rust_bindings_match_the_header():
    """rust/src/gpu/cuda/ffi.rs is generated from include/nne_cuda.h; a header change without a
    regenerated ffi.rs (or a hand edit of ffi.rs) fails here.  Also: one declaration per symbol."""
    import importlib.util
    gen_path = os.path.join(ROOT, "neural-network-engine_b200", "rust", "gen_ffi.py")
    spec = importlib.util.spec_from_file_location("gen_ffi", gen_path)
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    want = gen.generate(open(HEADER).read())
    have = open(gen.OUT).read()
    assert have == want, "ffi.rs is out of date: run neural-network-engine_b200/rust/gen_ffi.py"
    rust_syms = sorted(re.findall(r"pub fn (nne_\w+)\(", have))
    assert rust_syms == declared_symbols()


def test_rust_build_script_takes_every_kernel_file():
    """build.rs scans cuda/ instead of listing files, and every .cu of csrc/ is a kernel file the
    Makefile builds too (so the two build recipes cannot disagree about the file set)."""
    text = open(os.path.join(ROOT, "neural-network-engine_b200", "rust", "build.rs")).read()
    assert "read_dir(\"cuda\")" in text and ".cu\"" not in text.replace('x == "cu"', "")
    mk = open(os.path.join(ROOT, "neural-network-engine_b200", "csrc", "Makefile")).read()
    assert "$(wildcard *.cu)" in mk
