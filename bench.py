#!/usr/bin/env python
"""Headline benchmark: spiking ResNet-18 (T=4) inference throughput in images/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (fixed): spiking ResNet-18, T=4, global batch 512 sharded by batch over the N
ranks (strong scaling), 3x224x224 N(0,1) synthetic input with direct encoding, random-init
weights with BatchNorm folded, bf16 activations/weights with fp32 accumulation and fp32
LIF arithmetic, logits gathered over NCCL. One "step" is one forward pass of the whole
global batch.

Prints ONE JSON line (rank 0):
  value        images/s with the input batch already resident in HBM (CUDA-graph replay)
  e2e          images/s through the host-facing call: pinned host input -> device, forward,
               gather, logits -> host, every step
  roofline     the dominant kernel (the tcgen05 conv + LIF implicit GEMM): algorithmic
               FLOP / CUDA-event time of its launches, against the measured bf16 peak
  cpu_baseline the un-fused eager CPU path (oracle port of the reference's eager loop) on a
               small batch, on this host's cores
`--impl reference` times only that CPU path and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GLOBAL_BATCH = 512
T_STEPS = 4
IN_HW = (224, 224)
CLASSES = 1000


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), tf_burst=float(d["bf16_tflops"]),
                    tf_sustained=float(d["bf16_tflops_sustained"]), source="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def conv_flops(spec, shapes, B, T):
    """Algorithmic FLOP of each dense conv layer: 2 * T' * B * Ho*Wo * Cout * Cin*k*k, with T' = 1 for a
    layer fed by the (time-invariant) input frame, which is convolved once."""
    out = {}
    for L in spec:
        if L["op"] == "conv" and L["groups"] == 1:
            ho, wo, _ = shapes[L["dst"]]
            t_eff = 1 if L["src"] == "input" else T
            out[L["name"]] = 2.0 * t_eff * B * ho * wo * L["cout"] * L["cin"] * L["k"] * L["k"]
    return out


def cpu_eager_images_per_s(batch: int, reps: int, net: str = "resnet18", T: int = 4):
    """The reference's un-fused eager path on the host cores: the single-step model (conv -> BatchNorm -> LIF)
    called T times and averaged, fp32, with every LIF update done by the reference's own op
    (snn_custom.lif_forward_state of its runtime/snn_custom_ops.py, imported unmodified from the staged copy under
    oracle/_ref). Without that copy the oracle's port of the same loop runs instead. Uses every core this
    process may run on. Returns (images/s, threads, seconds per pass, kind)."""
    from triton_snn_fusion_b200 import specs   # plain-torch workload definition; loads no CUDA library

    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    spec = specs.NETS[net](CLASSES)
    params = specs.make_params(spec, seed=2026)
    x = torch.randn(batch, 3, *IN_HW, generator=torch.Generator().manual_seed(2026))
    ref_dir = ROOT / "oracle" / "_ref"
    if (ref_dir / "runtime" / "snn_custom_ops.py").exists():
        sys.dont_write_bytecode = True
        sys.path.insert(0, str(ref_dir))
        import runtime.snn_custom_ops as ref_ops   # the reference's file, with its own backends beneath it
        from oracle import torch_models
        ref_ops.configure_fused_op(backend="torch")
        model = torch_models.build(spec, params, T)

        def one_pass():
            model.layer.reset()
            return model(x)
        kind = "reference"
    else:
        from oracle import models as omodels

        def one_pass():
            return omodels.eager_forward(spec, params, x, T)
        kind = "port"
    with torch.no_grad():
        one_pass()  # warm-up
        times = []
        for _ in range(reps):
            t0 = time.perf_counter()
            one_pass()
            times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    return batch / med, torch.get_num_threads(), med, kind


def run_reference(args):
    """CPU arm: nothing of this library's CUDA code is loaded or run. One step = one timed pass over a bounded
    sample (batch 32) of the 512-image workload; images/s does not depend on the sample size."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    batch = 32
    reps = max(1, min(args.steps, 40))   # about 0.45 s per pass on 16 cores
    ips, cores, sec, kind = cpu_eager_images_per_s(batch, reps, args.net, args.T)
    sample = (f"{reps} timed passes of batch {batch} (a sample of the {args.global_batch}-image step), fp32, torch eager on "
              f"{cores} CPU threads, LIF by the reference's snn_custom.lif_forward_state" if kind == "reference" else
              f"{reps} timed passes of batch {batch} (a sample of the {args.global_batch}-image step), fp32, oracle port of "
              f"the eager loop on {cores} CPU threads")
    line = {
        "impl": "reference", "metric": metric_name(args.net, args.T), "value": ips, "unit": "images/s", "n_gpus": args.gpus,
        "steps": reps, "warmup": 1, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.T, args.global_batch, args.net), "parallelism": "cpu",
                   "images_per_step": batch},
        "cpu_baseline": {"value": ips, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": ips, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(net, T):
    return f"spiking_{net}_T{T}_images_per_sec"


def workload_name(T, batch, net="resnet18"):
    title = {"resnet18": "spiking ResNet-18", "mobilenet_v1": "spiking MobileNetV1"}[net]
    return f"{title} T={T}, global batch {batch}, 3x224x224 N(0,1), direct encoding"


def run_ours(args):
    import torch.distributed as dist
    global GLOBAL_BATCH, T_STEPS
    GLOBAL_BATCH = args.global_batch
    T_STEPS = args.T

    from triton_snn_fusion_b200 import _lib, nets
    from triton_snn_fusion_b200.parallel import gather_logits, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the fused kernels)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # the only collective is a 2 MB all-gather of logits per step: one NCCL block is plenty, and every SM it does
        # not occupy stays with the persistent conv grids (one block per SM) of the pass that runs meanwhile
        os.environ.setdefault("NCCL_MAX_CTAS", "1")
        os.environ.setdefault("NCCL_MIN_CTAS", "1")
        dist.init_process_group("nccl", device_id=dev)
    start, stop = shard_range(GLOBAL_BATCH, rank, world)
    B = stop - start
    K, Wm = args.steps, max(args.warmup, 3)

    spec = nets.NETS[args.net](CLASSES)
    params = nets.make_params(spec, seed=2026, gain=args.weight_gain)
    # this rank's shard of the seeded global batch, channels-last bf16, in pinned host memory
    g = torch.Generator().manual_seed(2026 + rank)
    host_in = torch.randn(B, *IN_HW, 3, generator=g).to(torch.bfloat16).pin_memory()

    def make_net():
        n = nets.CompiledNet(spec, params, batch=B, T=T_STEPS, in_hw=IN_HW, dtype=torch.bfloat16, device=dev,
                             conv_path=args.path)
        n.x_in.copy_(host_in)
        return n

    # `--in-flight` copies of the network take turns (pass i on copy i % copies, each on its own stream): the SMs one
    # pass leaves idle in the partly filled last wave of a layer run blocks of the other pass
    passes = nets.OverlappedPasses(make_net, copies=max(1, args.in_flight), graph=args.graph)
    net = passes.nets[0]
    copies = len(passes)
    host_out = [torch.empty(B, CLASSES, dtype=torch.float32).pin_memory() for _ in range(copies)]
    gathered = [torch.empty(GLOBAL_BATCH, CLASSES, dtype=torch.float32, device=dev) if world > 1 else None
                for _ in range(copies)]
    # The gather of a step's logits runs on a stream of its own, behind a copy of the logits: the pass that follows on
    # the same network copy does not wait for it (it only waits for the PREVIOUS gather of that copy before it
    # overwrites the staged logits), and the timed region ends after the last gather.
    comm = torch.cuda.Stream(dev) if world > 1 else None
    staged = [torch.empty(B, CLASSES, dtype=torch.float32, device=dev) if world > 1 else None for _ in range(copies)]
    gather_done = [torch.cuda.Event() for _ in range(copies)]

    def gather_after(logits, k):   # called inside copy k's stream
        if world == 1:
            return
        cur = torch.cuda.current_stream(dev)
        cur.wait_event(gather_done[k])
        staged[k].copy_(logits, non_blocking=True)
        ready = torch.cuda.Event()
        ready.record(cur)
        with torch.cuda.stream(comm):
            comm.wait_event(ready)
            gather_logits(staged[k], out=gathered[k])
            gather_done[k].record(comm)

    def step_resident(i):
        passes.run(i, then=gather_after)

    def step_e2e(i):
        # the user-facing call: pinned host batch in, fp32 logits out to pinned host memory. The copy of
        # a copy's next step (side stream, second staging buffer) overlaps the kernels of its current one; every
        # step's copies lie inside the timed region because the step's kernels wait for them.
        passes.submit(i, host_in, host_out[i % copies], then=gather_after)

    def timed(step_fn):
        for i in range(max(Wm, copies)):
            step_fn(i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        passes.fork()          # the copies' streams start after e0 ...
        for i in range(K):
            step_fn(i)
        passes.join()          # ... and e1 follows the last kernel of every copy
        if comm is not None:
            torch.cuda.current_stream(dev).wait_stream(comm)   # ... and the last gather
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / K

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_resident = timed(step_resident)
    ms_e2e = timed(step_e2e)
    clocks = sampler.stop() if rank == 0 else None

    # ---- per-layer device times (un-graphed, CUDA events on the launching stream), after the timed region
    stream = torch.cuda.current_stream(dev).cuda_stream
    reps = 5
    layer_ms, layer_launches = {}, {}
    for fn, a, name in net._calls:
        for _ in range(2):
            fn(*a, stream)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn(*a, stream)
        e1.record()
        torch.cuda.synchronize()
        layer_ms[name] = layer_ms.get(name, 0.0) + e0.elapsed_time(e1) / reps   # a layer runs once per window of T
        layer_launches[name] = layer_launches.get(name, 0) + 1
    status = _lib.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = _peaks()
    flops = conv_flops(spec, net.shapes, B, T_STEPS)
    # which kernel serves which layer: the library's own dispatch, asked through its query entry point
    def kernel_of(L):
        if L["op"] != "conv":
            return {"maxpool": "maxpool3x3s2", "head": "avgpool_linear_mean", "tail": "lif_avgpool_linear"}[L["op"]]
        if L["groups"] != 1:
            return "dwconv3x3_lif"
        if L["cin"] == 3 and L["k"] == 7:
            return "stem (s2d + stem_gemm_lif)"
        hi, wi, _ = net.shapes[L["src"]]
        name = _lib.conv_kernel_name(T_STEPS, B, L["cin"], hi, wi, L["cout"], L["k"], L["s"], L["p"], torch.bfloat16,
                                     one_frame=(L["cin"] == 3), residual=bool(L.get("residual")))
        return name + (" (3-channel stem)" if L["cin"] == 3 else "")
    by_kernel = {}
    fused_into = {D["name"]: consumer for consumer, D in net.fused_sc.items()}   # shortcut conv -> the launch it rides in
    by_name = {L["name"]: L for L in spec}
    for L in spec:
        if L["name"] in fused_into:   # no launch of its own: its flops count for the consumer's kernel
            by_kernel.setdefault(kernel_of(by_name[fused_into[L["name"]]]),
                                 {"launches": 0, "ms": 0.0, "flop": 0.0})["flop"] += flops.get(L["name"], 0.0)
            continue
        k = kernel_of(L)
        e = by_kernel.setdefault(k, {"launches": 0, "ms": 0.0, "flop": 0.0})
        e["launches"] += layer_launches[L["name"]]
        e["ms"] += layer_ms[L["name"]]
        e["flop"] += flops.get(L["name"], 0.0)
        if k == "dwconv3x3_lif":   # HBM-bound: input frames + spikes out + the membrane written once, 16-bit each
            hi, wi, _ = net.shapes[L["src"]]
            ho, wo, co = net.shapes[L["dst"]]
            e["bytes"] = e.get("bytes", 0.0) + 2.0 * (T_STEPS * B * co * (hi * wi + ho * wo) + B * co * ho * wo)
    total_ms = sum(layer_ms.values())
    dom = max(by_kernel, key=lambda k: by_kernel[k]["ms"])
    d = by_kernel[dom]
    achieved = d["flop"] / (d["ms"] * 1e-3) / 1e12 if d["ms"] > 0 else 0.0
    top = sorted(layer_ms.items(), key=lambda kv: -kv[1])[:6]
    # DRAM traffic per launch of the dominant kernel: one ncu capture of a 128->128, 56x56, T=4, batch-32
    # layer read 103.17 MB and wrote 78.43 MB (its ncu summary is committed with the other profiles). The kernel
    # moves each activation once, so the figure is scaled by the activation elements (in + out) of the
    # layers it serves here and averaged over its launches.
    traffic = None
    if dom == "conv3x3_pair":
        cap_bytes, cap_elems = 181.60e6, 4 * 32 * 56 * 56 * (128 + 128)
        elems = 0
        for L in spec:
            if L["name"] not in fused_into and kernel_of(L) == dom:
                ho, wo, co = net.shapes[L["dst"]]
                hi, wi, _ = net.shapes[L["src"]]
                elems += T_STEPS * B * (hi * wi * L["cin"] + ho * wo * (co + (co if L.get("residual") else 0)))
        traffic = cap_bytes * elems / cap_elems / d["launches"]
    bound, peak, unit, peak_src = "tensor", peaks["tf_sustained"], "TFLOP/s", peaks["source"] + " (sustained bf16)"
    if d.get("bytes"):
        bound, peak, unit, peak_src = "hbm", peaks["hbm"], "GB/s", peaks["source"] + " (copy bandwidth)"
        achieved = d["bytes"] / (d["ms"] * 1e-3) / 1e9
    roofline = {
        "kernel": f"{dom} ({d['launches']} launches per step)",
        "bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
        "frac": achieved / peak, "peak_source": peak_src,
        "traffic": traffic, "traffic_unit": "bytes per launch (ncu capture of one layer, scaled by activation elements)",
        "share_of_step": d["ms"] / total_ms if total_ms else None,
        "kernels": {k: {"launches": v["launches"], "ms": round(v["ms"], 3), "share": round(v["ms"] / total_ms, 3),
                        "tflops": round(v["flop"] / (v["ms"] * 1e-3) / 1e12, 1) if v["flop"] else None}
                    for k, v in sorted(by_kernel.items(), key=lambda kv: -kv[1]["ms"])},
        "top_layers_ms": {k: round(v, 4) for k, v in top},
    }
    if args.layers:
        print(json.dumps({"layers_ms": {k: round(v, 4) for k, v in layer_ms.items()}}), file=sys.stderr)
    cpu_batch = 32   # 24 timed passes: about 10 s of CPU work on 16 cores
    ips_cpu, cores, sec, cpu_kind = (cpu_eager_images_per_s(cpu_batch, 24 if T_STEPS <= 4 else 12, args.net, T_STEPS)
                                     if world == 1 and not args.no_cpu else (None, None, None, None))
    line = {
        "metric": metric_name(args.net, T_STEPS), "value": GLOBAL_BATCH / (ms_resident * 1e-3), "unit": "images/s", "n_gpus": world,
        "steps": K, "warmup": Wm, "ms_per_step": ms_resident, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(T_STEPS, GLOBAL_BATCH, args.net),
                   "parallelism": f"batch-sharded x{world}", "per_gpu_batch": B, "cuda_graph": bool(args.graph),
                   "passes_in_flight": copies, "conv_path": args.path,
                   "l2": "no flush needed: each step streams >3 GB of activations per GPU, far beyond the 126 MB L2"},
        "e2e": {"value": GLOBAL_BATCH / (ms_e2e * 1e-3), "unit": "images/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": host_in.numel() * host_in.element_size() * world,
                "d2h_bytes_per_step": host_out[0].numel() * host_out[0].element_size() * world},
        "gpu_launches": net.launches_per_forward * K,
        "roofline": roofline,
        "clocks": clocks,
        "device_status": status,
    }
    if ips_cpu is not None:
        line["cpu_baseline"] = {"value": ips_cpu, "unit": "images/s", "cores": cores, "kind": cpu_kind,
                                "sample": f"timed passes of batch {cpu_batch} of the same network, fp32 torch eager "
                                          f"(conv->BN->LIF per timestep, T calls of the single-step model), "
                                          f"{sec:.2f} s per pass"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--T", type=int, default=4, help="timesteps (the headline is T = 4; 8 runs as two windows of four)")
    ap.add_argument("--net", default="resnet18", choices=["resnet18", "mobilenet_v1"],
                    help="network (the headline is resnet18; mobilenet_v1 is the depthwise / pointwise workload)")
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "tcgen05", "tcgen05_taps", "tcgen05_halo"])
    ap.add_argument("--no-graph", dest="graph", action="store_false")
    ap.add_argument("--in-flight", type=int, default=2,
                    help="forward passes in flight (copies of the network on their own streams that take turns)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--layers", action="store_true", help="also print every layer's device time to stderr")
    ap.add_argument("--weight-gain", type=float, default=1.0,
                    help="scale the conv weights of all but the first layer (1.0 = the benchmark's initialisation, with "
                         "which the deeper stages barely spike; > 1 keeps every stage spiking, to show that the timing "
                         "does not depend on the spike values)")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH,
                    help="images per step over all ranks (the benchmark's configuration is 512; other values are for "
                         "studying how the kernels behave at the per-GPU batch of an N-GPU run)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
