"""Layer specs of the benchmark networks and their seeded parameters (plain torch, no GPU library).

A network is a list of dict specs: ``conv`` (dense or depthwise conv + BatchNorm, optionally + residual,
optionally + LIF), ``maxpool``, ``tail`` (LIF -> global avgpool -> linear) and ``head`` (avgpool -> linear on
spikes). The executor (``nets.CompiledNet``) and the CPU checkers both read these lists; this module imports
nothing but torch so that a CPU-only process can build the same workload without loading the CUDA library.
BatchNorm folding follows the reference's rewrite (compiler/fx_lif_rewrite.py:340-353 in
pengjh0111/triton-snn-fusion).
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

LIF = dict(v_th=1.0, v_reset=0.0, tau=2.0)


# ------------------------------------------------------------------ specs ----
def _conv(name, src, dst, cin, cout, k, s, p, groups=1, residual=None, lif=True):
    return dict(op="conv", name=name, src=src, dst=dst, cin=cin, cout=cout, k=k, s=s, p=p, groups=groups,
                residual=residual, lif=lif)


def spiking_cnn_small(num_classes: int = 10) -> List[dict]:
    """conv3x3 3->64 s1, 64->128 s2, 128->256 s2 (each + BN + LIF), then LIF -> avgpool -> linear."""
    return [
        _conv("conv1", "input", "a1", 3, 64, 3, 1, 1),
        _conv("conv2", "a1", "a2", 64, 128, 3, 2, 1),
        _conv("conv3", "a2", "a3", 128, 256, 3, 2, 1),
        dict(op="tail", name="tail", src="a3", cin=256, classes=num_classes),
    ]


def spiking_mobilenet_v1(num_classes: int = 1000) -> List[dict]:
    """Width-1.0 MobileNetV1: stem conv3x3 s2 32, 13 depthwise/pointwise blocks, LIF -> avgpool -> linear."""
    spec = [_conv("stem", "input", "s0", 3, 32, 3, 2, 1)]
    plan = [(64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2)] + [(512, 1)] * 5 + [(1024, 2), (1024, 1)]
    cin, src = 32, "s0"
    for i, (cout, s) in enumerate(plan):
        spec.append(_conv(f"dw{i}", src, f"d{i}", cin, cin, 3, s, 1, groups=cin))
        spec.append(_conv(f"pw{i}", f"d{i}", f"p{i}", cin, cout, 1, 1, 0))
        cin, src = cout, f"p{i}"
    spec.append(dict(op="tail", name="tail", src=src, cin=cin, classes=num_classes))
    return spec


def spiking_resnet18(num_classes: int = 1000) -> List[dict]:
    """7x7 s2 stem + BN + LIF, maxpool, 8 basic blocks (conv-BN-LIF, conv-BN-add-LIF) with identity or
    1x1-s2 conv+BN shortcuts, avgpool + linear averaged over T."""
    spec = [_conv("stem", "input", "s0", 3, 64, 7, 2, 3), dict(op="maxpool", name="pool", src="s0", dst="x0", c=64)]
    cin, src = 64, "x0"
    for stage, cout in enumerate((64, 128, 256, 512)):
        for blk in range(2):
            s = 2 if (stage > 0 and blk == 0) else 1
            tag = f"l{stage + 1}b{blk}"
            spec.append(_conv(f"{tag}.conv1", src, f"{tag}.y", cin, cout, 3, s, 1))
            if s != 1 or cin != cout:
                spec.append(_conv(f"{tag}.down", src, f"{tag}.sc", cin, cout, 1, s, 0, lif=False))
                res = f"{tag}.sc"
            else:
                res = src
            spec.append(_conv(f"{tag}.conv2", f"{tag}.y", f"{tag}.out", cout, cout, 3, 1, 1, residual=res))
            cin, src = cout, f"{tag}.out"
    spec.append(dict(op="head", name="fc", src=src, cin=cin, classes=num_classes))
    return spec


NETS = {"cnn_small": spiking_cnn_small, "mobilenet_v1": spiking_mobilenet_v1, "resnet18": spiking_resnet18}


# ------------------------------------------------------------- parameters ----
def make_params(spec: List[dict], seed: int = 2026, gain: float = 1.0) -> Dict[str, Dict[str, torch.Tensor]]:
    """Seeded fp32 CPU parameters: Kaiming-normal conv / linear weights, BN gamma U(0.5,1.5),
    beta N(0,0.1), running mean N(0,0.1), running var U(0.5,1.5). With this initialisation a deep
    spiking net falls silent after a few layers (timing does not depend on it; parity tests of whole
    networks want spikes everywhere): ``gain`` > 1 scales the conv weights of all but the first layer."""
    g = torch.Generator().manual_seed(seed)
    params: Dict[str, Dict[str, torch.Tensor]] = {}
    for L in spec:
        if L["op"] == "conv":
            fan_in = (L["cin"] // L["groups"]) * L["k"] * L["k"]
            c = L["cout"]
            params[L["name"]] = dict(
                w=torch.randn(c, L["cin"] // L["groups"], L["k"], L["k"], generator=g) * math.sqrt(2.0 / fan_in)
                * (gain if L["src"] != "input" else 1.0),
                gamma=torch.rand(c, generator=g) + 0.5,
                beta=torch.randn(c, generator=g) * 0.1,
                mean=torch.randn(c, generator=g) * 0.1,
                var=torch.rand(c, generator=g) + 0.5,
            )
        elif L["op"] in ("tail", "head"):
            params[L["name"]] = dict(
                w=torch.randn(L["classes"], L["cin"], generator=g) * math.sqrt(2.0 / L["cin"]),
                b=torch.randn(L["classes"], generator=g) * 0.01,
            )
    return params


def fold_bn(w, gamma, beta, mean, var, eps: float = 1e-5):
    """BatchNorm (inference) folded into a bias-free conv, as the reference's rewrite does
    (compiler/fx_lif_rewrite.py:340-353): scale = gamma / sqrt(var + eps); W' = W * scale;
    b' = (0 - mean) * scale + beta."""
    scale = gamma / torch.sqrt(var + float(eps))
    return w * scale.reshape(-1, 1, 1, 1), (torch.zeros_like(mean) - mean) * scale + beta


def folded_params(spec, params, dtype) -> Dict[str, Dict[str, torch.Tensor]]:
    """BN-folded parameters rounded to the compute dtype (CPU tensors, torch layouts)."""
    out = {}
    for L in spec:
        p = params.get(L["name"])
        if p is None:
            continue
        if L["op"] == "conv":
            w, b = fold_bn(p["w"], p["gamma"], p["beta"], p["mean"], p["var"])
            out[L["name"]] = dict(w=w.to(dtype), b=b.to(dtype))
        else:
            out[L["name"]] = dict(w=p["w"].to(dtype), b=p["b"].to(dtype))
    return out
