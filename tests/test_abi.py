"""The C-ABI library loads and exports every symbol include/tc_b200.h declares (no compute calls)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "tc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tc_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = _declared_functions()
    for must in ("tc_plan_create", "tc_plan_set_extents", "tc_plan_commit", "tc_execute", "tc_execute_host",
                 "tc_plan_destroy", "tc_status_string", "tc_expr_describe"):
        assert must in names


def test_library_exports_every_declared_symbol(pkg):
    handle = ctypes.CDLL(pkg.LIB_PATH)
    for name in _declared_functions():
        assert hasattr(handle, name), "libtc_b200.so does not export %s" % name


def test_python_bindings_cover_the_header(pkg):
    assert sorted(pkg.exported_symbols()) == _declared_functions()


def test_status_strings_and_version(pkg):
    lib = pkg.lib()
    assert lib.tc_status_string(0) == b"ok"
    for s in range(1, 10):
        assert lib.tc_status_string(s) not in (b"", b"unknown status")
    assert lib.tc_status_string(99) == b"unknown status"
    assert b"sm_100a" in lib.tc_version()


def test_null_arguments_are_rejected(pkg):
    lib = pkg.lib()
    out = ctypes.c_void_p()
    assert lib.tc_plan_create(None, 0, None, ctypes.byref(out)) == 2
    assert lib.tc_plan_create(b"t3 [a,2] += sum(b,2) * t2 [b,a] * v2 [b];", 7, None, ctypes.byref(out)) == 2
    assert lib.tc_plan_commit(None) == 2
    assert lib.tc_execute(None, None, None, None, None) == 2
    assert lib.tc_plan_launches(None) == -1
    lib.tc_plan_destroy(None)  # no-op


def test_product_never_links_the_checker(pkg):
    """The shipped library must not depend on anything under oracle/."""
    data = open(pkg.LIB_PATH, "rb").read()
    assert b"tc_oracle_contract" not in data and b"liboracle" not in data
    for f in os.listdir(os.path.join(ROOT, "cgo2019-ae_b200")):
        if f.endswith(".py"):
            src = open(os.path.join(ROOT, "cgo2019-ae_b200", f)).read()
            assert "oracle" not in src, f
