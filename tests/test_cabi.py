"""CPU: the C-ABI library loads, exports every symbol include/intfa.h declares, its ctypes mirror
matches the C struct layout, and argument validation answers before anything touches a device."""
import ctypes
import importlib
import os
import re
import subprocess
import sys

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "intfa.h")


@pytest.fixture(scope="module")
def lib():
    L = importlib.import_module("int-flashattention_b200._lib")
    if not os.path.exists(L.LIB_PATH):
        importlib.import_module("int-flashattention_b200.build").build()
    return L


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(intfa_\w+)\s*\(", src)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 9
    handle = lib.load()
    for n in names:
        assert hasattr(handle, n), n
    assert sorted(lib.EXPORTS) == [n for n in names if n in lib.EXPORTS]
    missing_in_binding = [n for n in names if n not in lib.EXPORTS]
    assert missing_in_binding == [], missing_in_binding


def test_struct_layout_matches_header(lib, tmp_path):
    fields = [f[0] for f in lib.IntfaFwdParams._fields_]
    c = ['#include <stdio.h>', '#include <stddef.h>', '#include "intfa.h"', 'int main(void){',
         'printf("%zu\\n", sizeof(IntfaFwdParams));']
    c += ['printf("%%zu\\n", offsetof(IntfaFwdParams, %s));' % f for f in fields]
    c += ['return 0;}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(c))
    exe = tmp_path / "layout"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    nums = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    assert nums[0] == ctypes.sizeof(lib.IntfaFwdParams)
    for f, off in zip(fields, nums[1:]):
        assert getattr(lib.IntfaFwdParams, f).offset == off, f


def test_version_and_error_text(lib):
    h = lib.load()
    assert h.intfa_version() >= 100
    assert h.intfa_fwd(None, None) == lib.ERR_INVALID_ARG
    assert "NULL" in lib.last_error()


def test_validation_rejects_before_launch(lib):
    h = lib.load()
    P = lib.IntfaFwdParams()
    P.B, P.H, P.Nq, P.Nk, P.D, P.G = 1, 1, 128, 128, 48, 64
    assert h.intfa_fwd(ctypes.byref(P), None) == lib.ERR_UNSUPPORTED       # head_dim 48: not one of 16, 32, 64, 128, 256
    assert "head_dim" in lib.last_error()
    P.D, P.G, P.variant = 256, 128, lib.VARIANT_HALF
    assert h.intfa_fwd(ctypes.byref(P), None) == lib.ERR_UNSUPPORTED       # half-int8 at head_dim 256: G = 64 only
    P.variant = lib.VARIANT_FULL
    P.D = 128
    P.Nq = 100
    assert h.intfa_fwd(ctypes.byref(P), None) == lib.ERR_INVALID_ARG       # a ragged Nq is fine; q is NULL
    P.Nq = 128
    P.G = 96
    assert h.intfa_fwd(ctypes.byref(P), None) == lib.ERR_UNSUPPORTED       # G must be 64 or 128
    P.D, P.G = 128, 128
    assert h.intfa_fwd(ctypes.byref(P), None) == lib.ERR_INVALID_ARG       # q is NULL
    P.H, P.H_kv = 8, 3
    assert h.intfa_fwd(ctypes.byref(P), None) == lib.ERR_INVALID_ARG       # query heads not a multiple of K/V heads
    assert "H_kv" in lib.last_error()
    P.H_kv = 2
    P.o_dtype = 5
    assert h.intfa_fwd(ctypes.byref(P), None) == lib.ERR_INVALID_ARG       # unknown output type
    assert "o_dtype" in lib.last_error()
    P.o_dtype = 0
    P.variant = 7
    assert h.intfa_fwd(ctypes.byref(P), None) == lib.ERR_INVALID_ARG
    assert h.intfa_quant_pertoken(None, None, None, None, 1, 1, 1, 128, None) == lib.ERR_INVALID_ARG
    assert h.intfa_quant_v_workspace_bytes(2, 3, 128) == 2 * 3 * 128 * 4


def test_python_surface_refuses_cpu_tensors(pkg):
    import torch
    q = torch.zeros(1, 1, 128, 64, dtype=torch.int8)
    s = torch.ones(1, 1, 128)
    with pytest.raises(RuntimeError, match="CUDA"):
        pkg.attention_full_int8(q, q, q, s, s, torch.ones(1, 1), False, 1.0)
    with pytest.raises(RuntimeError, match="CUDA"):
        pkg.quant_pertoken(torch.zeros(1, 1, 128, 64, dtype=torch.float16))
    with pytest.raises(AssertionError):     # the reference's own head-dim assertion
        pkg.attention_int8(torch.zeros(1, 1, 128, 48, dtype=torch.int8), q, q.half(), s, s, False, 1.0)


def test_product_package_never_imports_the_oracle():
    pkg_dir = os.path.join(ROOT, "int-flashattention_b200")
    pat = re.compile(r"^\s*(from|import)\s+\S*oracle", re.M)
    for dirpath, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith(".py"):
                assert not pat.search(open(os.path.join(dirpath, f)).read()), f
