"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    src = open(os.path.join(ROOT, "include", "b200gpt2.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    src = re.sub(r"typedef[^;]*\(\s*\*[^;]*;", "", src)  # function-pointer typedefs are not exports
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}]*\)\s*;", src)
    return sorted(set(n for n in names if n not in ("defined",)))


def test_header_declares_the_reference_entry_points():
    names = _declared_functions()
    for required in ("matmul_forward", "attention_forward", "layernorm_forward", "fused_residual_layernorm_forward",
                     "fused_residual_layernorm", "residual_forward", "gelu_forward", "encoder_forward",
                     "b200_gpt2_forward"):
        assert required in names


def test_library_exports_every_declared_symbol(pkg):
    import __graft_entry__ as ge
    ge.build()
    lib = ctypes.CDLL(pkg.LIB_PATH)
    missing = [n for n in _declared_functions() if not hasattr(lib, n)]
    assert not missing, missing
    assert set(pkg.EXPORTS) <= set(_declared_functions())


def test_status_strings_and_host_only_entry_points(pkg):
    lib = pkg.lib()
    assert lib.b200_status_string(0) == b"ok"
    assert b"16-byte" in lib.b200_status_string(3)
    cfg = pkg.GPT2_124M.c()
    offs = (ctypes.c_size_t * 17)()
    total = lib.b200_gpt2_param_offsets(ctypes.byref(cfg), offs)
    assert total == 124475904 and list(offs) == pkg.param_offsets(pkg.GPT2_124M)
    # NULL handling that needs no device
    assert lib.b200_ctx_destroy(None) == 1
    assert lib.b200_matmul_forward(None, None, None, None, None, 1, 1, 4, 4, 0, None, 0) == 1


def test_missing_library_fails_loudly(pkg, monkeypatch):
    import pytest
    monkeypatch.setattr(pkg, "_lib", None)
    monkeypatch.setattr(pkg, "LIB_PATH", "/nonexistent/libb200gpt2.so")
    with pytest.raises(pkg.B200Error, match="missing"):
        pkg.lib()
