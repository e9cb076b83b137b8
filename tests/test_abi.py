"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import re

from conftest import ROOT


def _declared_symbols():
    text = (ROOT / "include" / "snnb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(snnb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    from triton_snn_fusion_b200 import _lib

    names = _declared_symbols()
    assert len(names) >= 10
    raw = ctypes.CDLL(str(_lib.LIB_PATH))
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/snnb200.h but not exported"
    # the Python binding covers the same set
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_text():
    from triton_snn_fusion_b200 import _lib

    assert _lib.lib.snnb_version() >= 100
    # argument validation happens on the host, before any CUDA call
    st = _lib.lib.snnb_lif_scan(None, None, None, None, 4, 16, 0, 0, 0, 1.0, 0.0, 2.0, None)
    assert st == 1
    assert b"null pointer" in _lib.lib.snnb_last_error()
