"""The CPU oracle reproduces the golden vectors recorded from the reference, bit for bit."""
import ctypes
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import ROOT, golden_cases, load_golden
from oracle import snn_oracle as orc


@pytest.mark.parametrize("name", golden_cases("lif"))
def test_lif(name):
    a, z = load_golden(name)
    s, v = orc.temporal_lif(z["x"], z["v_init"], a["v_th"], a["v_reset"], a["tau"])
    assert torch.equal(s, z["spikes"]) and torch.equal(v, z["v"])


@pytest.mark.parametrize("name", golden_cases("conv"))
def test_conv(name):
    a, z = load_golden(name)
    xs = list(z["x"])
    res = list(z["residual"]) if "residual" in z else None
    s, v = orc.temporal_conv_lif(xs, z["w"], z["b"], z["v_init"], [a["stride"]] * 2, [a["padding"]] * 2, [1, 1],
                                 a["groups"], a["v_th"], a["v_reset"], a["tau"], residuals=res)
    assert torch.equal(s, z["spikes"]) and torch.equal(v, z["v"])


@pytest.mark.parametrize("name", golden_cases("linear"))
def test_linear(name):
    a, z = load_golden(name)
    s, v = orc.temporal_linear_lif(z["x"], z["w"], z.get("b"), z["v_init"], a["v_th"], a["v_reset"], a["tau"])
    assert torch.equal(s, z["spikes"]) and torch.equal(v, z["v"])


@pytest.mark.parametrize("name", golden_cases("tail"))
def test_tail(name):
    a, z = load_golden(name)
    o, v = orc.temporal_lif_avgpool_linear(z["x"], z["v_init"], z["w"], z["b"], a["v_th"], a["v_reset"], a["tau"])
    assert torch.equal(o, z["out_sum"]) and torch.equal(v, z["v"])


def test_fold_bn():
    a, z = load_golden("fold_bn")
    w, b = orc.fold_bn(z["w"], None, z["mean"], z["var"], z["gamma"], z["beta"], a["eps"])
    assert torch.equal(w, z["w_folded"]) and torch.equal(b, z["b_folded"])


def _c_oracle():
    so = ROOT / "oracle" / "_build" / "liblif_oracle.so"
    if not so.exists():
        import subprocess
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    lib = ctypes.CDLL(str(so))
    lib.lif_scan_f32.restype = None
    lib.lif_scan_f32.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_int64] + [ctypes.c_float] * 3
    return lib


@pytest.mark.parametrize("name", golden_cases("lif"))
def test_c_oracle_lif(name):
    """The plain-C restatement of the scan agrees with the reference's vectors too."""
    a, z = load_golden(name)
    lib = _c_oracle()
    x = z["x"].contiguous()
    T, n = x.shape[0], x[0].numel()
    v0 = z["v_init"].contiguous() if z["v_init"].dim() else None
    s = torch.empty_like(x)
    v = torch.empty_like(x[0])
    lib.lif_scan_f32(x.data_ptr(), v0.data_ptr() if v0 is not None else None, s.data_ptr(), v.data_ptr(),
                     T, n, a["v_th"], a["v_reset"], a["tau"])
    assert torch.equal(s, z["spikes"]) and torch.equal(v, z["v"])
