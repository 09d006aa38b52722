"""CPU: the C-ABI shared library loads and exports every symbol include/b200moe.h declares.
No compute entry point is called here (there is no GPU)."""
import ctypes
import os
import re

import util  # noqa: F401  (path setup)
from justgoal_b200 import _lib

HEADER = os.path.join(util.ROOT, "include", "b200moe.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z_0-9]+)\s*\(", src)))


def test_header_declares_the_operator():
    names = declared_functions()
    for must in ("b200moe_create", "b200moe_destroy", "b200moe_workspace_bytes", "b200moe_forward",
                 "b200moe_forward_routed", "b200moe_ep_combine", "b200moe_route", "b200moe_status"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_strerror_and_struct_sizes():
    assert b"workspace" in _lib.lib.b200moe_strerror(-2)
    assert _lib.lib.b200moe_strerror(0) == b"ok"
    assert ctypes.sizeof(_lib.Config) == 8 * 4
    assert ctypes.sizeof(_lib.WsLayout) == 23 * ctypes.sizeof(ctypes.c_size_t)


def test_null_arguments_are_rejected_without_a_device():
    assert _lib.lib.b200moe_create(None, None) == -1
    assert _lib.lib.b200moe_destroy(None) == -1
    assert _lib.lib.b200moe_workspace_bytes(None, 4, None) == -1
