"""CPU tests of the C-ABI boundary: the library builds, loads, exports every
symbol the public header declares, and rejects bad arguments before touching a
GPU.  No kernel is launched here."""
import ctypes as C
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sspmm_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:sspmm|svc|smtx)_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for n in ("sspmm_f16_f32", "sspmm_f16_f16", "sspmm_f16_f16_batched", "svc_begin", "svc_finish", "svc_free",
              "sspmm_sorted_row_swizzle", "sspmm_last_error_string"):
        assert n in names


def test_library_exports_every_declared_symbol(lib):
    from sspmm_b200 import capi
    for n in declared_functions():
        assert hasattr(lib, n), n
        assert n in capi.SIGNATURES, f"{n} has no ctypes signature"
    assert set(capi.SIGNATURES) == set(declared_functions())


def test_cxx_overloads_are_exported(lib):
    # the link-level drop-in: the six overloads of include/sspmm.cuh, by their Itanium names
    from sspmm_b200 import build
    out = subprocess.run(["nm", "-D", "--defined-only", build.LIB_PATH], capture_output=True, text=True).stdout
    for sym in ("_ZN4spmm5SSpMMEiiiiPKiS1_S1_PK6__halfS4_Pf", "_ZN4spmm5SSpMMEiiiiPKiS1_S1_PK6__halfS4_PS2_",
                "_ZN4spmm5SSpMMEiiiiPKiS1_S1_PKfS3_Pf", "_ZN4spmm4SpMMEiiiiPKiS1_S1_PK6__halfS4_Pf",
                "_ZN4spmm4SpMMEiiiiPKiS1_S1_PK6__halfS4_PS2_", "_ZN4spmm4SpMMEiiiiPKiS1_S1_PKfS3_Pf"):
        assert sym in out, sym


def test_header_compiles_as_c():
    r = subprocess.run(["gcc", "-std=c99", "-fsyntax-only", "-x", "c", HEADER], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_argument_validation_without_gpu(lib):
    assert lib.sspmm_f16_f32(4, 7, 64, 64, None, None, None, None, None, None, None) == 1
    assert b"vec_length" in lib.sspmm_last_error_string()
    assert lib.sspmm_f16_f16(-1, 8, 64, 64, None, None, None, None, None, None, None) == 1
    assert lib.sspmm_f16_f16(4, 8, 64, 64, None, None, None, None, None, None, None) == 1
    assert b"null" in lib.sspmm_last_error_string()
    # empty problems succeed without any launch
    assert lib.sspmm_f16_f16(0, 8, 64, 64, None, None, None, None, None, None, None) == 0
    assert lib.sspmm_f16_f16(4, 16, 0, 64, None, None, None, None, None, None, None) == 0
    job, nvec = C.c_void_p(), C.c_int64()
    assert lib.svc_begin(8, 8, 5, None, None, None, None, C.byref(job), C.byref(nvec)) == 1
    assert lib.svc_begin(8, 1 << 30, 8, None, None, None, None, C.byref(job), C.byref(nvec)) == 1
    assert b"exceeds" in lib.sspmm_last_error_string()
    assert lib.sspmm_set_kernel(9) == 1
    assert lib.sspmm_set_kernel(4) == 0
    assert lib.sspmm_set_kernel(5) == 0
    assert lib.sspmm_set_kernel(6) == 1
    assert lib.sspmm_set_kernel(0) == 0
    assert lib.sspmm_version().startswith(b"sspmm_b200")


def test_float_overload_matches_reference_behaviour(lib, capfd):
    # SSpMM/src/sspmm.cu:651-661: prints and returns cudaSuccess, launches nothing
    fn = getattr(lib, "_ZN4spmm5SSpMMEiiiiPKiS1_S1_PKfS3_Pf")
    fn.restype = C.c_int
    assert fn(1, 8, 64, 64, None, None, None, None, None, None) == 0


def test_python_ops_refuse_cpu_tensors():
    import torch
    from sspmm_b200 import ops
    t = torch.zeros(3, dtype=torch.int32)
    with pytest.raises(ValueError):
        ops.sspmm(t, t, torch.zeros(8, dtype=torch.float16), torch.zeros(4, 8, dtype=torch.float16), 8)
