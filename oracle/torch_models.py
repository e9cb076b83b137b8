"""Single-step ``nn.Module`` versions of the benchmark networks — TEST INFRASTRUCTURE ONLY.

The reference's compile pipeline starts from an ordinary single-step spiking model whose neurons are
stateful modules that call ``torch.ops.snn_custom.lif_forward_state`` (its own benchmark takes such a
node from a ``test`` package that is not part of its checkout, and the network definitions from
SpikingJelly; benchmarks/validate_chronos_baselines.py:17-18, :87). This module supplies both for the
layer specs of ``triton_snn_fusion_b200.specs``: a stateful LIF node with the reference's conventions
and a module that runs a spec one timestep at a time, plus the T-step loop wrapper of the reference's
single-step mode (benchmarks/validate_chronos_baselines.py:234-244: call the model T times on the same
input and average).

Importing the reference's ``runtime.snn_custom_ops`` (which registers the ``snn_custom`` ops) is the
caller's job: the tests and the CPU baseline do it from the staged copy under ``oracle/_ref``.
"""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.nn as nn
import torch.nn.functional as F


class StatefulLIF(nn.Module):
    """LIF neuron that keeps its membrane between calls. The first call of a sequence starts from
    ``zeros_like(x)``, which is the form the reference's matchers recognise as "zero initial state"
    (compiler/fx_lif_rewrite.py:111-114), and the ``.default`` overload is the one they compare against
    (compiler/fx_lif_rewrite.py:71-72)."""

    def __init__(self, v_th: float = 1.0, v_reset: float = 0.0, tau: float = 2.0):
        super().__init__()
        self.v_th, self.v_reset, self.tau = float(v_th), float(v_reset), float(tau)
        self.v = None

    def reset(self) -> None:
        self.v = None

    def forward(self, x):
        if self.v is None:
            self.v = torch.zeros_like(x)
        spike, self.v = torch.ops.snn_custom.lif_forward_state.default(x, self.v, self.v_th, self.v_reset, self.tau, False)
        return spike


def _key(name: str) -> str:
    return name.replace(".", "_")


class SpecNet(nn.Module):
    """One timestep of a layer spec: conv -> BatchNorm (eval) -> [+ residual] -> [LIF] per ``conv`` entry."""

    def __init__(self, spec: List[dict], params: Dict[str, Dict[str, torch.Tensor]], eps: float = 1e-5):
        super().__init__()
        self.spec = spec
        self.convs, self.bns, self.lifs = nn.ModuleDict(), nn.ModuleDict(), nn.ModuleDict()
        self.fc = None
        for L in spec:
            p = params.get(L["name"])
            k = _key(L["name"])
            if L["op"] == "conv":
                conv = nn.Conv2d(L["cin"], L["cout"], L["k"], L["s"], L["p"], groups=L["groups"], bias=False)
                bn = nn.BatchNorm2d(L["cout"], eps=eps)
                with torch.no_grad():
                    conv.weight.copy_(p["w"])
                    bn.weight.copy_(p["gamma"]); bn.bias.copy_(p["beta"])
                    bn.running_mean.copy_(p["mean"]); bn.running_var.copy_(p["var"])
                self.convs[k], self.bns[k] = conv, bn
                if L["lif"]:
                    self.lifs[k] = StatefulLIF()
            elif L["op"] in ("tail", "head"):
                self.fc = nn.Linear(L["cin"], L["classes"])
                with torch.no_grad():
                    self.fc.weight.copy_(p["w"]); self.fc.bias.copy_(p["b"])
                if L["op"] == "tail":
                    self.lifs[k] = StatefulLIF()
        self.eval()

    def reset(self) -> None:
        for m in self.lifs.values():
            m.reset()

    def forward(self, x):
        acts = {"input": x}
        out = None
        for L in self.spec:
            k = _key(L["name"])
            h = acts[L["src"]]
            if L["op"] == "conv":
                y = self.bns[k](self.convs[k](h))
                if L.get("residual"):
                    y = y + acts[L["residual"]]
                acts[L["dst"]] = self.lifs[k](y) if L["lif"] else y
            elif L["op"] == "maxpool":
                acts[L["dst"]] = F.max_pool2d(h, 3, 2, 1)
            elif L["op"] == "tail":
                out = self.fc(torch.flatten(F.adaptive_avg_pool2d(self.lifs[k](h), 1), 1))
            elif L["op"] == "head":
                out = self.fc(torch.flatten(F.adaptive_avg_pool2d(h, 1), 1))
        return out


class SingleStepLoop(nn.Module):
    """T calls of a single-step model on the same input, averaged (direct encoding)."""

    def __init__(self, layer: nn.Module, T: int):
        super().__init__()
        self.layer, self.T = layer, int(T)

    def forward(self, x):
        total = 0
        for _ in range(self.T):
            total = total + self.layer(x)
        return total / self.T


def build(spec, params, T: int) -> SingleStepLoop:
    return SingleStepLoop(SpecNet(spec, params), T)
