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


def test_kernel_choice_is_reported_without_a_gpu():
    """snnb_conv_lif_which mirrors the dispatch of snnb_conv_lif on the host: the ResNet-18 / MobileNet layer shapes
    land on the kernels the design assigns them."""
    import torch
    from triton_snn_fusion_b200 import _lib
    bf = torch.bfloat16
    name = _lib.conv_kernel_name
    assert name(4, 8, 128, 56, 56, 128, 3, 1, 1, bf) == "conv3x3_pair"
    assert name(8, 8, 64, 56, 56, 64, 3, 1, 1, bf, residual=True) == "conv3x3_pair"      # any even T
    assert name(4, 8, 64, 56, 56, 128, 3, 2, 1, bf) == "conv3x3_pair"                    # stride 2 through phase views
    assert name(4, 8, 32, 112, 112, 64, 1, 1, 0, bf) == "conv3x3_pair"                   # partial channel slab
    assert name(4, 8, 512, 7, 7, 512, 3, 1, 1, bf) == "conv3x3_pair"                     # two images per tile
    assert name(3, 8, 64, 14, 14, 64, 3, 1, 1, bf) == "conv3x3_halo"                     # odd T
    assert name(4, 8, 64, 28, 28, 128, 1, 2, 0, bf) == "conv_lif_tc"                     # strided 1x1
    assert name(4, 8, 3, 224, 224, 32, 3, 2, 1, bf, one_frame=True) == "conv3x3_smallcin"
    assert name(4, 8, 64, 28, 28, 64, 3, 1, 1, torch.float32) == "conv_lif_simt"          # fp32: CUDA cores
    import pytest
    with pytest.raises(_lib.SnnbError, match="no tensor-core kernel"):
        name(4, 8, 24, 13, 11, 40, 5, 1, 2, bf, path=_lib.PATH_TCGEN05)
