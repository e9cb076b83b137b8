"""CPU oracle for whole networks — TEST INFRASTRUCTURE ONLY (see snn_oracle.py).

Runs a layer spec of ``triton_snn_fusion_b200.nets`` the way the reference's un-fused
eager baseline runs a model: every layer evaluated per timestep as conv -> BatchNorm ->
LIF with plain torch ops (the reference's ``baseline_single_step_mode_eager``,
benchmarks/benchmark_chronos_runtime.py:281-289, wrapper
benchmarks/validate_chronos_baselines.py:234-244; LIF node arithmetic
runtime/snn_custom_ops.py:384-409), logits averaged over T. The layer-major loop order
used here visits the same (layer, t) pairs as the reference's t-major loop and every
value depends only on earlier t of the same layer and on the layer below, so the
results are identical.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from . import snn_oracle as orc

LIF = dict(v_th=1.0, v_reset=0.0, tau=2.0)


def eager_forward(spec: List[dict], params, x: torch.Tensor, T: int, eps: float = 1e-5):
    """Un-fused eager path with un-folded BatchNorm, fp32. x: [B,3,H,W]. Returns logits [B,classes]."""
    acts: Dict[str, List[torch.Tensor]] = {"input": [x] * T}
    logits = None
    for L in spec:
        xs = acts[L["src"]]
        if L["op"] == "conv":
            p = params[L["name"]]
            res = acts[L["residual"]] if L.get("residual") else None
            v = None
            out = []
            for t in range(T):
                y = F.conv2d(xs[t], p["w"], None, L["s"], L["p"], 1, L["groups"])
                y = F.batch_norm(y, p["mean"], p["var"], p["gamma"], p["beta"], False, 0.0, eps)
                if res is not None:
                    y = y + res[t]
                if L["lif"]:
                    y, v = orc.lif_step(y, v, **LIF)
                out.append(y)
            acts[L["dst"]] = out
        elif L["op"] == "maxpool":
            acts[L["dst"]] = [F.max_pool2d(a, 3, 2, 1) for a in xs]
        elif L["op"] == "tail":
            p = params[L["name"]]
            total, _ = orc.temporal_lif_avgpool_linear(torch.stack(xs), None, p["w"], p["b"], **LIF)
            logits = total / T
        elif L["op"] == "head":
            p = params[L["name"]]
            logits = sum(F.linear(F.adaptive_avg_pool2d(a, 1).flatten(1), p["w"], p["b"]) for a in xs) / T
    return logits


def folded_forward(spec: List[dict], folded, x: torch.Tensor, T: int,
                   teacher: Optional[Dict[str, torch.Tensor]] = None):
    """Fused-op semantics on the CPU with BN-folded parameters (any dtype, widened to fp32).

    Returns (logits, layers) where layers[name] = (spikes [T,B,C,H,W], v [B,C,H,W]) for LIF convs or
    (values, None) otherwise. With ``teacher`` (name -> [T,B,C,H,W] activations produced by the
    device), every layer reads the teacher's version of its inputs, so one layer's spike flips do
    not propagate into the comparison of the next.
    """
    x = orc.widen(x)
    acts: Dict[str, torch.Tensor] = {"input": torch.stack([x] * T)}
    layers = {}
    logits = None

    def src_of(name):
        if teacher is not None and name in teacher:
            return orc.widen(teacher[name])
        return acts[name]

    for L in spec:
        xs = src_of(L["src"])
        if L["op"] == "conv":
            p = folded[L["name"]]
            w, b = orc.widen(p["w"]), orc.widen(p["b"])
            res = list(src_of(L["residual"])) if L.get("residual") else None
            if L["lif"]:
                s, v = orc.temporal_conv_lif(list(xs), w, b, None, [L["s"]] * 2, [L["p"]] * 2, [1, 1], L["groups"],
                                             LIF["v_th"], LIF["v_reset"], LIF["tau"], residuals=res)
            else:
                s, v = orc.temporal_conv_only(list(xs), w, b, [L["s"]] * 2, [L["p"]] * 2, 1, L["groups"]), None
                if res is not None:
                    s = s + torch.stack(res)
            acts[L["dst"]] = s
            layers[L["name"]] = (s, v)
        elif L["op"] == "maxpool":
            acts[L["dst"]] = torch.stack([F.max_pool2d(a, 3, 2, 1) for a in xs])
            layers[L["name"]] = (acts[L["dst"]], None)
        elif L["op"] == "tail":
            p = folded[L["name"]]
            total, v = orc.temporal_lif_avgpool_linear(xs, None, orc.widen(p["w"]), orc.widen(p["b"]), **LIF)
            logits = total / T
            layers[L["name"]] = (logits, v)
        elif L["op"] == "head":
            p = folded[L["name"]]
            w, b = orc.widen(p["w"]), orc.widen(p["b"])
            logits = sum(F.linear(F.adaptive_avg_pool2d(a, 1).flatten(1), w, b) for a in xs) / T
            layers[L["name"]] = (logits, None)
    return logits, layers
