"""The C-ABI library loads without a GPU and exports every function the header declares."""
import ctypes
import os
import re

from strata_b200 import library_path, load_library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "strata_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(strata_moe_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported():
    names = declared_functions()
    assert len(names) >= 20
    lib = ctypes.CDLL(library_path())
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_knows_every_export():
    from strata_b200.api import EXPORTS
    assert set(declared_functions()) == set(EXPORTS)
    load_library()


def test_create_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        return
    lib = load_library()
    h = ctypes.c_void_p()
    assert lib.strata_moe_create(0, None, ctypes.byref(h)) != 0 and not h.value
