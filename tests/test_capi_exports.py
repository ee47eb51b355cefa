"""CPU checks of the drop-in boundary: the shared library loads without a GPU and exports every symbol the
header declares; argument checking works without touching a device."""
import ctypes as C
import os
import re

from xstar_moe import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            text = re.sub(r"/\*.*?\*/", "", open(os.path.join(inc, f)).read(), flags=re.S)
            names |= set(re.findall(r"\b(xs_moe_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    L = capi.lib()
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), f"{n} is declared under include/ but not exported"
    assert sorted(capi.EXPORTS) == names, "the ctypes binding and the header list different entry points"


def test_status_strings_and_argument_checks_need_no_gpu():
    L = capi.lib()
    assert L.xs_moe_status_string(0) == b"ok"
    assert L.xs_moe_status_string(-6) == b"device-side wait timed out"
    cfg = capi.make_config(8, 256, 8, 2, 128, 0)
    n = C.c_size_t(0)
    assert L.xs_moe_workspace_bytes(C.byref(cfg), C.byref(n)) == 0 and n.value > 8 * 2 * 256 * 4
    bad = capi.make_config(8, 256, 8, 0, 128, 0)
    assert L.xs_moe_workspace_bytes(C.byref(bad), C.byref(n)) == -1
    assert b"top_k out of range" in L.xs_moe_last_error()
    bad = capi.make_config(8, 256, 8, 2, 128, 0, local_begin=4, local_count=8)
    assert L.xs_moe_workspace_bytes(C.byref(bad), C.byref(n)) == -1
    assert b"expert count mismatch" in L.xs_moe_last_error()
    bad = capi.make_config(8, 256, 8, 2, 128, 0, routed_format=7)
    assert L.xs_moe_workspace_bytes(C.byref(bad), C.byref(n)) == -2
    assert b"unsupported dtype" in L.xs_moe_last_error()


def test_workspace_grows_with_tokens():
    a = capi.workspace_bytes(capi.make_config(1, 4096, 256, 6, 2048, 1))
    b = capi.workspace_bytes(capi.make_config(128, 4096, 256, 6, 2048, 1))
    assert b > a > 0
