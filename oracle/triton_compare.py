"""Times the reference's own Triton kernels next to this library's kernels on the same GPU.

    python oracle/triton_compare.py [--reps 20] [--only lif,linear,tail,conv]

TEST / MEASUREMENT INFRASTRUCTURE ONLY: the reference's kernel modules are imported unmodified from the staged
copy under oracle/_ref (oracle/stage_ref.py) and JIT-compiled by Triton for the GPU at hand; nothing here is used
by the library. For each workload the reference launcher and this library's entry point are called on identical
seeded inputs, the results are compared (spike flip rate), and both are timed with CUDA events after warm-up
(the reference's first calls include JIT compilation and autotuning, which the warm-up absorbs). Workloads:

  lif     standalone temporal LIF scan, T=4, N = 2^24, fp32           kernels/generated_temporal_lif_kernel.py:98-154
  linear  temporal linear + LIF, T=4, M=4096, K=768, N=3072, fp16      kernels/generated_temporal_linear_lif_kernel.py:205-363
  tail    LIF -> avgpool -> linear, [4,256,1024,7,7] -> 1000, fp16      kernels/generated_temporal_lif_avgpool_linear_kernel.py:120-209
  conv    conv3x3 + LIF, T=4, batch 64, 128 -> 128, 56x56, fp16         runtime/triton_convlif_backend.py:393-430 (its kernel
          generator imports SpikingJelly at module level; an empty stand-in module is registered for that import)

The reference accepts fp32 and fp16 only (its support gates reject bf16), so the 16-bit cases run in fp16 on both
sides. One JSON line per workload; a reference kernel that cannot be compiled or run is reported with its error
text instead of a time.
"""
from __future__ import annotations

import argparse
import json
import sys
import types
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref"
DEV = "cuda"
LIF = (1.0, 0.0, 2.0)


def _time(fn, reps, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def _flips(a, b):
    return float((a.float() != b.float()).float().mean())


def _report(name, shape, ours_ms, ref_fn, reps, check):
    line = {"workload": name, "shape": shape, "ours_ms": round(ours_ms, 4)}
    try:
        out = ref_fn()
        torch.cuda.synchronize()
        line["check"] = check(out)
        line["reference_triton_ms"] = round(_time(ref_fn, reps), 4)
        line["speedup"] = round(line["reference_triton_ms"] / ours_ms, 2)
    except Exception as exc:   # the comparison is best effort: say why the reference kernel did not run
        line["reference_triton_error"] = f"{type(exc).__name__}: {str(exc)[:300]}"
    print(json.dumps(line), flush=True)


def case_lif(reps):
    from kernels.generated_temporal_lif_kernel import run_fused_temporal_lif_state_kernel as ref
    from triton_snn_fusion_b200.runtime.triton_temporal_lif_backend import run_triton_fused_temporal_lif_state as ours
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(4, 64, 64, 64, 64, device=DEV, generator=g) * 0.8 + 0.6     # [T, N, C, H, W], 2^24 per step
    z = torch.tensor(0.0, device=DEV)
    mine = ours(x, z, *LIF, False, strict=True)
    ms = _time(lambda: ours(x, z, *LIF, False, strict=True), reps)
    _report("lif_scan T4 n=2^24 fp32", list(x.shape), ms, lambda: ref(x, z, *LIF, False), reps,
            lambda out: {"spike_flip_rate": _flips(out[0], mine.spikes), "bit_exact": bool(torch.equal(out[0], mine.spikes))})


def case_linear(reps):
    from kernels.generated_temporal_linear_lif_kernel import run_fused_temporal_linear_lif_state_kernel as ref
    from triton_snn_fusion_b200.runtime.triton_temporal_linear_lif_backend import (
        run_triton_fused_temporal_linear_lif_state_packed as ours)
    dt = torch.float16
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.rand(4, 4096, 768, device=DEV, generator=g) < 0.15).to(dt)
    w = (torch.randn(3072, 768, device=DEV, generator=g) * 768 ** -0.5 * 2.5).to(dt)
    b = torch.zeros(3072, device=DEV, dtype=dt)
    z = torch.tensor(0.0, device=DEV, dtype=dt)
    mine = ours(x, w, b, z, *LIF, False, strict=True)
    ms = _time(lambda: ours(x, w, b, z, *LIF, False, strict=True), reps)
    _report("linear_lif T4 M4096 K768 N3072 fp16", [4, 4096, 768, 3072], ms, lambda: ref(x, w, b, z, *LIF, False), reps,
            lambda out: {"spike_flip_rate": _flips(out[0], mine.spikes)})


def case_tail(reps):
    from kernels.generated_temporal_lif_avgpool_linear_kernel import run_fused_temporal_lif_avgpool_linear_kernel as ref
    from triton_snn_fusion_b200.runtime.triton_temporal_lif_avgpool_linear_backend import (
        run_triton_fused_temporal_lif_avgpool_linear as ours)
    dt = torch.float16
    g = torch.Generator(device=DEV).manual_seed(0)
    x_nchw = (torch.randn(4, 256, 1024, 7, 7, device=DEV, generator=g) * 0.75 + 0.15).to(dt)
    x_nhwc = x_nchw.permute(0, 1, 3, 4, 2).contiguous().permute(0, 1, 4, 2, 3)   # this library's layout between layers
    w = (torch.randn(1000, 1024, device=DEV, generator=g) * 0.05).to(dt)
    b = torch.zeros(1000, device=DEV, dtype=dt)
    z = torch.tensor(0.0, device=DEV, dtype=dt)
    mine = ours(x_nhwc, z, w, b, *LIF, False, strict=True)
    ms = _time(lambda: ours(x_nhwc, z, w, b, *LIF, False, strict=True), reps)
    _report("lif_avgpool_linear [4,256,1024,7,7]->1000 fp16", list(x_nchw.shape), ms,
            lambda: ref(x_nchw, z, w, b, *LIF, False), reps,
            lambda out: {"max_abs_logit_diff": float((out[0].float() - mine.out_sum.float()).abs().max()),
                         "membrane_equal": bool(torch.equal(out[1], mine.v_next.contiguous()))})


def case_conv(reps):
    # the reference's conv kernel generator imports SpikingJelly (absent here) for its own self-test classes; the
    # kernels themselves do not use it
    for name in ("spikingjelly", "spikingjelly.activation_based"):
        sys.modules.setdefault(name, types.ModuleType(name))
    ab = sys.modules["spikingjelly.activation_based"]
    for attr in ("functional", "layer", "neuron", "surrogate"):
        if not hasattr(ab, attr):
            setattr(ab, attr, types.ModuleType(f"spikingjelly.activation_based.{attr}"))
    from triton_snn_fusion_b200.runtime.triton_convlif_backend import run_triton_fused_temporal_conv_lif_state as ours
    dt = torch.float16
    g = torch.Generator(device=DEV).manual_seed(0)
    xs = [(torch.rand(64, 128, 56, 56, device=DEV, generator=g) < 0.15).to(dt) for _ in range(4)]
    xs_cl = [x.contiguous(memory_format=torch.channels_last) for x in xs]
    w = (torch.randn(128, 128, 3, 3, device=DEV, generator=g) * (2.0 / 1152) ** 0.5 * 2.5).to(dt)
    b = (torch.randn(128, device=DEV, generator=g) * 0.1).to(dt)
    z = torch.tensor(0.0, device=DEV, dtype=dt)
    args = ([1, 1], [1, 1], [1, 1], 1, *LIF, False)
    mine = ours(xs_cl, w, b, z, *args, strict=True)
    ms = _time(lambda: ours(xs_cl, w, b, z, *args, strict=True), reps)

    def ref_fn():
        import importlib
        be = importlib.import_module("runtime.triton_convlif_backend")   # the reference's own module (no install())
        return be.run_triton_fused_temporal_conv_lif_state(xs, w, b, z, *args, strict=True, compute_dtype="float16")

    _report("conv3x3_lif T4 B64 128->128 56x56 fp16", [4, 64, 128, 56, 56], ms, ref_fn, reps,
            lambda out: {"spike_flip_rate": _flips(out.spikes, mine.spikes)})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--only", default="lif,linear,tail,conv")
    a = ap.parse_args()
    if not (REF / "kernels").is_dir():
        raise SystemExit("the reference is not staged: python oracle/stage_ref.py --reference <checkout>")
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(REF))
    sys.path.insert(0, str(ROOT))
    import os
    os.environ.setdefault("TRITON_CACHE_DIR", "/tmp/triton_cache_ref")
    cases = {"lif": case_lif, "linear": case_linear, "tail": case_tail, "conv": case_conv}
    for name in a.only.split(","):
        try:
            cases[name](a.reps)
        except Exception as exc:
            print(json.dumps({"workload": name, "error": f"{type(exc).__name__}: {str(exc)[:300]}"}), flush=True)


if __name__ == "__main__":
    main()
