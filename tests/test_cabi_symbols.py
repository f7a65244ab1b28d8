"""The C-ABI library builds, loads without a GPU and exports every symbol that
include/b200_lora.h declares (no compute call is made here)."""

import ctypes
import os
import re

from nanovllm_voxcpm_b200 import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_lora.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#ifdef B200_TRACE.*?#endif", "", text, flags=re.S)  # entry point of the tuning build only
    return sorted(set(re.findall(r"\b(lora_b200_\w+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = ctypes.CDLL(N.LIB_PATH)
    declared = _declared_symbols()
    assert "lora_b200_add" in declared and "lora_b200_version" in declared
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/b200_lora.h but not exported"


def test_binding_covers_header():
    assert sorted(N.exported_symbols()) == _declared_symbols()


def test_version_and_error_string():
    lib = N.lib()
    assert lib.lora_b200_version() == N.ABI_VERSION
    assert isinstance(lib.lora_b200_last_error(), bytes)


def test_bad_arguments_are_rejected_before_any_launch():
    """Status codes come back without touching the GPU (null pointers, bad sizes)."""
    lib = N.lib()
    rc = lib.lora_b200_add(None, 8, None, 8, 4, 8, 1, None, None, None, None, 1, 8, None, None, None, None, None,
                           None, None, 0, 1.0, N.DT_BF16, N.IMPL_AUTO, None, 0, None)
    assert rc == N.E_INVAL
    assert b"null" in lib.lora_b200_last_error()
    rc = lib.lora_b200_add(None, 8, None, 8, 4, 8, 1, None, None, None, None, 1, 8, None, None, None, None, None,
                           None, None, 0, 1.0, 77, N.IMPL_AUTO, None, 0, None)
    assert rc == N.E_INVAL and b"dtype" in lib.lora_b200_last_error()
    # T == 0 is a valid empty call
    rc = lib.lora_b200_add(None, 8, None, 8, 0, 8, 1, None, None, None, None, 1, 8, None, None, None, None, None,
                           None, None, 0, 1.0, N.DT_BF16, N.IMPL_AUTO, None, 0, None)
    assert rc == 0
