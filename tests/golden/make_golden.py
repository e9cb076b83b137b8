"""Generates the golden vectors under tests/golden/ from the reference itself.

Run where a checkout of pengjh0111/triton-snn-fusion is available:

    python tests/golden/make_golden.py --reference <path to the checkout>

For every case it builds seeded CPU inputs (input distributions follow the
reference's own kernel checks, e.g. benchmarks/benchmark_temporal_lif_kernel.py:72-77),
evaluates the reference's ``*_torch`` functions of runtime/snn_custom_ops.py
(imported unmodified from the checkout), requires the restatement in
``oracle/snn_oracle.py`` to reproduce them bit for bit, and writes inputs and
reference outputs to ``<case>.npz``. ``index.json`` lists the cases with their
scalar arguments. The vectors are small (a few KB each) and committed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import snn_oracle as orc  # noqa: E402


def _import_reference(path: str):
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    sys.dont_write_bytecode = True
    sys.path.insert(0, path)
    import runtime.snn_custom_ops as ref_ops  # type: ignore
    from compiler.fx_lif_rewrite import fold_bn_into_conv_params  # type: ignore

    return ref_ops, fold_bn_into_conv_params


def _np(t):
    return t.detach().cpu().numpy()


LIF_VARIANTS = [
    # name, v_th, v_reset, tau
    ("hard_tau2", 1.0, 0.0, 2.0),
    ("soft_tau2", 1.0, -1.0, 2.0),
    ("hard_tau3", 1.0, 0.0, 3.0),
    ("hard_tau1", 1.0, 0.0, 1.0),
    ("hard_th05_reset01_tau4", 0.5, 0.1, 4.0),
]


def gen_lif(ref_ops, out: dict):
    for T in (1, 4, 5):
        for vname, v_th, v_reset, tau in LIF_VARIANTS:
            for with_v in (False, True):
                shape = (2, 3, 5, 7)
                torch.manual_seed(2026 + T + shape[1])
                x = torch.randn((T,) + shape) * 0.75 + 0.15
                v0 = torch.randn(shape) * 0.4 if with_v else torch.tensor(0.0)
                rs, rv = ref_ops.fused_temporal_lif_state_torch(x, v0, v_th, v_reset, tau, False)
                ms, mv = orc.temporal_lif(x, v0, v_th, v_reset, tau)
                assert torch.equal(rs, ms) and torch.equal(rv, mv), ("lif", T, vname, with_v)
                name = f"lif_T{T}_{vname}_{'v' if with_v else 'z'}"
                out[name] = dict(kind="lif", args=dict(v_th=v_th, v_reset=v_reset, tau=tau),
                                 arrays=dict(x=_np(x), v_init=_np(v0), spikes=_np(rs), v=_np(rv)))


CONV_CASES = [
    # name, Cin, Cout, k, stride, pad, groups, H, W
    ("k3_s1_p1", 8, 16, 3, 1, 1, 1, 9, 7),
    ("k3_s2_p1", 8, 16, 3, 2, 1, 1, 10, 8),
    ("k3_s2_p1_odd", 4, 8, 3, 2, 1, 1, 9, 7),
    ("k1_s1_p0", 8, 16, 1, 1, 0, 1, 6, 5),
    ("k7_s2_p3", 3, 8, 7, 2, 3, 1, 16, 14),
    ("depthwise_k3_s1_p1", 8, 8, 3, 1, 1, 8, 9, 7),
    ("depthwise_k3_s2_p1", 8, 8, 3, 2, 1, 8, 10, 7),
]


def gen_conv(ref_ops, out: dict):
    T, B = 4, 2
    for name, cin, cout, k, s, p, g, H, W in CONV_CASES:
        for residual in (False, True):
            for vname, v_th, v_reset, tau in (LIF_VARIANTS[0], LIF_VARIANTS[1]):
                torch.manual_seed(2026 + T + cin + cout + k + s)
                xs = [torch.randn(B, cin, H, W) for _ in range(T)]
                w = torch.randn(cout, cin // g, k, k) * (2.0 / (cin // g * k * k)) ** 0.5
                b = torch.randn(cout) * 0.1
                ho = (H + 2 * p - k) // s + 1
                wo = (W + 2 * p - k) // s + 1
                v0 = torch.randn(B, cout, ho, wo) * 0.3 if vname.startswith("soft") else torch.tensor(0.0)
                stride, pad, dil = [s, s], [p, p], [1, 1]
                if residual:
                    res = [torch.randn(B, cout, ho, wo) * 0.5 for _ in range(T)]
                    rs, rv = ref_ops.fused_temporal_conv_add_lif_state_torch(
                        xs, res, w, b, v0, stride, pad, dil, g, v_th, v_reset, tau, False)
                else:
                    res = None
                    rs, rv = ref_ops.fused_temporal_conv_lif_state_torch(
                        xs, w, b, v0, stride, pad, dil, g, v_th, v_reset, tau, False)
                ms, mv = orc.temporal_conv_lif(xs, w, b, v0, stride, pad, dil, g, v_th, v_reset, tau, residuals=res)
                assert torch.equal(rs, ms) and torch.equal(rv, mv), ("conv", name, residual, vname)
                arrays = dict(x=_np(torch.stack(xs)), w=_np(w), b=_np(b), v_init=_np(v0), spikes=_np(rs), v=_np(rv))
                if residual:
                    arrays["residual"] = _np(torch.stack(res))
                out[f"conv_{name}_{'res' if residual else 'plain'}_{vname}"] = dict(
                    kind="conv", args=dict(stride=s, padding=p, groups=g, v_th=v_th, v_reset=v_reset, tau=tau),
                    arrays=arrays)


def gen_linear(ref_ops, out: dict):
    for T, M, K, N, with_bias in ((4, 5, 24, 16, True), (2, 7, 64, 32, False), (1, 3, 8, 8, True)):
        torch.manual_seed(2026 + T + M + K + N)
        x = torch.randn(T, M, K) * 0.5
        w = torch.randn(N, K) * (1.0 / K) ** 0.5
        b = torch.randn(N) * 0.1 if with_bias else None
        for vname, v_th, v_reset, tau in (LIF_VARIANTS[0], LIF_VARIANTS[1], LIF_VARIANTS[2]):
            v0 = torch.randn(M, N) * 0.3 if vname.startswith("soft") else torch.tensor(0.0)
            b_ref = b if b is not None else torch.empty(0)
            rs, rv = ref_ops.fused_temporal_linear_lif_state_packed_torch(x, w, b_ref, v0, v_th, v_reset, tau, False)
            ms, mv = orc.temporal_linear_lif(x, w, b, v0, v_th, v_reset, tau)
            assert torch.equal(rs, ms) and torch.equal(rv, mv), ("linear", T, M, K, N, vname)
            arrays = dict(x=_np(x), w=_np(w), v_init=_np(v0), spikes=_np(rs), v=_np(rv))
            if b is not None:
                arrays["b"] = _np(b)
            out[f"linear_T{T}_M{M}_K{K}_N{N}_{vname}"] = dict(
                kind="linear", args=dict(v_th=v_th, v_reset=v_reset, tau=tau), arrays=arrays)


def gen_tail(ref_ops, out: dict):
    for T, N, C, H, W, K in ((4, 2, 8, 3, 3, 5), (2, 3, 16, 7, 7, 10), (1, 1, 4, 2, 5, 3)):
        torch.manual_seed(2026 + T + N + C + K)
        x = torch.randn(T, N, C, H, W) * 0.75 + 0.15
        w = torch.randn(K, C) * 0.05
        b = torch.randn(K) * 0.05
        for vname, v_th, v_reset, tau in (LIF_VARIANTS[0], LIF_VARIANTS[1]):
            v0 = torch.randn(N, C, H, W) * 0.3 if vname.startswith("soft") else torch.tensor(0.0)
            ro, rv = ref_ops.fused_temporal_lif_avgpool_linear_torch(x, v0, w, b, v_th, v_reset, tau, False)
            mo, mv = orc.temporal_lif_avgpool_linear(x, v0, w, b, v_th, v_reset, tau)
            assert torch.equal(ro, mo) and torch.equal(rv, mv), ("tail", T, N, C, vname)
            out[f"tail_T{T}_N{N}_C{C}_K{K}_{vname}"] = dict(
                kind="tail", args=dict(v_th=v_th, v_reset=v_reset, tau=tau),
                arrays=dict(x=_np(x), w=_np(w), b=_np(b), v_init=_np(v0), out_sum=_np(ro), v=_np(rv)))


def gen_fold_bn(fold_ref, out: dict):
    torch.manual_seed(2026)
    cout, cin, k = 8, 4, 3
    w = torch.randn(cout, cin, k, k)
    gamma = torch.rand(cout) + 0.5
    beta = torch.randn(cout) * 0.1
    mean = torch.randn(cout) * 0.1
    var = torch.rand(cout) + 0.5
    rw, rb = fold_ref(w, None, mean, var, gamma, beta, 1e-5)
    mw, mb = orc.fold_bn(w, None, mean, var, gamma, beta, 1e-5)
    assert torch.equal(rw, mw) and torch.equal(rb, mb)
    out["fold_bn"] = dict(kind="fold_bn", args=dict(eps=1e-5),
                          arrays=dict(w=_np(w), gamma=_np(gamma), beta=_np(beta), mean=_np(mean), var=_np(var),
                                      w_folded=_np(rw), b_folded=_np(rb)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of pengjh0111/triton-snn-fusion")
    ns = ap.parse_args()
    ref_ops, fold_ref = _import_reference(ns.reference)
    cases: dict = {}
    gen_lif(ref_ops, cases)
    gen_conv(ref_ops, cases)
    gen_linear(ref_ops, cases)
    gen_tail(ref_ops, cases)
    gen_fold_bn(fold_ref, cases)
    index = {}
    for name, case in cases.items():
        np.savez_compressed(HERE / f"{name}.npz", **case["arrays"])
        index[name] = dict(kind=case["kind"], args=case["args"])
    (HERE / "index.json").write_text(json.dumps(
        dict(torch=torch.__version__, generator="tests/golden/make_golden.py", cases=index), indent=1, sort_keys=True))
    total = sum((HERE / f"{n}.npz").stat().st_size for n in cases)
    print(f"{len(cases)} cases, {total / 1024:.1f} KiB; oracle/snn_oracle.py matches the reference bit for bit on all")


if __name__ == "__main__":
    main()
