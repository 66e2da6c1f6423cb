"""CPU: the C-ABI library loads, exports every symbol include/b200moe.h declares, and its
host-side argument checks answer with status codes (no GPU work is attempted here)."""
import ctypes
import os
import re

import pytest

import gfx1151_engine_b200 as pkg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = pkg.lib()
    names = header_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), "libb200moe.so does not export " + n
    # the ctypes table in the package covers the same set
    assert sorted(pkg.SYMBOLS) == names


def test_version_and_status_strings():
    assert pkg.version().startswith("b200moe ") and "sm_100a" in pkg.version()
    L = pkg.lib()
    assert L.b200moe_status_string(0) == b"ok"
    assert L.b200moe_status_string(5) == b"device-side wait timed out"
    assert L.b200moe_status_string(99) == b"unknown status"


def _create(**kw):
    base = dict(experts=8, topk=2, d_model=128, d_mid=64, n_layers=1, max_tokens=4, has_shared=0,
                device=0, gemm_impl=0, decode_max_tokens=0, ep_rank=0, ep_size=1, ep_sm_margin=0, decode_impl=0)
    base.update(kw)
    cfg = pkg.Config(*[base[n] for n, _ in pkg.Config._fields_[:-1]])
    h = ctypes.c_void_p()
    return pkg.lib().b200moe_create(ctypes.byref(cfg), ctypes.byref(h)), h


@pytest.mark.parametrize("kw,status", [
    (dict(experts=0), 1), (dict(topk=0), 1), (dict(max_tokens=0), 1), (dict(ep_rank=2, ep_size=2), 1),
    (dict(experts=1024), 2), (dict(topk=17, experts=32), 2), (dict(d_model=100), 2), (dict(d_mid=96), 2),
    (dict(experts=8, topk=9), 2), (dict(experts=9, ep_size=2), 2),
])
def test_create_rejects_bad_configs(kw, status):
    st, h = _create(**kw)
    assert st == status and not h.value


def test_null_arguments():
    L = pkg.lib()
    assert L.b200moe_create(None, None) == 1
    assert L.b200moe_destroy(None) == 1
    assert L.b200moe_forward(None, 0, None, 1, None, None, None) == 1
    assert L.b200moe_launch_count(None) == 0
    assert L.b200moe_last_error(None) == b"null handle"


def test_missing_library_raises(monkeypatch, tmp_path):
    """No fallback: a missing .so is an ImportError naming the build command."""
    monkeypatch.setattr(pkg, "_lib", None)
    monkeypatch.setattr(pkg, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no fallback"):
        pkg.lib()
