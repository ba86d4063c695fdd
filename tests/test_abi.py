"""CPU: the C-ABI library loads and exports every entry point the header declares; argument
errors come back as a status plus a message, never as a crash.  No compute call is made."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    import __graft_entry__ as ge
    ge.build()
    return ge.load_package()


def header_symbols():
    names = set()
    for f in os.listdir(os.path.join(ROOT, "include")):
        if f.endswith(".h"):
            text = open(os.path.join(ROOT, "include", f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text))
    return names


def test_every_declared_symbol_is_exported(built):
    lib = C.CDLL(built.library_path())
    syms = header_symbols()
    assert len(syms) >= 20
    for s in syms:
        assert hasattr(lib, s), f"{s} is declared in include/ but not exported"
    from importlib import import_module
    L = import_module("mlx_rs_b200._lib")
    assert set(L.EXPORTS) == syms, "the ctypes binding table and the header differ"


def test_errors_are_reported_not_fatal(built):
    lib = built.lib()
    seen = []
    HANDLER = C.CFUNCTYPE(None, C.c_char_p, C.c_void_p)
    cb = HANDLER(lambda msg, data: seen.append(msg.decode()))
    lib.b200_set_error_handler(C.cast(cb, C.c_void_p), None, None)
    try:
        h = C.c_void_p()
        import torch
        if not torch.cuda.is_available():
            rc = lib.b200_ctx_create(C.byref(h), 0)       # no device here: must fail cleanly
            assert rc != 0 and lib.b200_last_error()
        rc = lib.b200_ctx_create(None, 0)
        assert rc != 0 and b"out is null" in lib.b200_last_error()
        rc = lib.b200_quantize(None, None, 0, 1, 64, 64, 4, None, None, None, None)
        assert rc != 0 and b"context is null" in lib.b200_last_error()
        assert seen and "context is null" in seen[-1]
        assert lib.b200_ctx_destroy(None) == 0
        assert lib.b200_ctx_launch_count(None) == 0
    finally:
        lib.b200_set_error_handler(None, None, None)


def test_package_refuses_to_run_without_gpu(built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(built.B200Error):
        built.Context()
