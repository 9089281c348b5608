"""The C-ABI library loads and exports every entry point include/unica_b200.h declares (no GPU needed: no compute call)."""

import ctypes
import re

from conftest import ROOT


def declared() -> set[str]:
    text = (ROOT / "include" / "unica_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(unica_b200_\w+)\s*\(", text))


def test_library_builds_and_exports_the_header():
    from unicaattention_b200 import build, lib

    path = build.build()
    handle = ctypes.CDLL(str(path))
    names = declared()
    assert len(names) >= 7
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in include/unica_b200.h but not exported"
    assert set(lib.SIGNATURES) <= names, "the Python binding names an entry point the header does not declare"
    assert lib.library().unica_b200_version() >= 1


def test_argument_errors_need_no_gpu():
    """Argument checks come before any CUDA call, raise ValueError and leave a message."""
    import pytest

    from unicaattention_b200 import lib

    layout = lib.TokenLayout(0, 0, 128, 1)
    with pytest.raises(ValueError, match="null pointer"):
        lib.call("unica_b200_quantize_int8", None, layout, None, 1, 64, 64, 1, None, None, None)
    with pytest.raises(ValueError, match="block_tokens"):
        lib.call("unica_b200_quantize_int8", ctypes.c_void_p(16), layout, None, 1, 64, 32, 2, ctypes.c_void_p(16),
                 ctypes.c_void_p(16), None)
    with pytest.raises(ValueError, match="multiple of 256"):
        lib.call("unica_b200_channel_stats", *[ctypes.c_void_p(16), layout, 1, 64, 100], *[ctypes.c_void_p(16)] * 4, None)
