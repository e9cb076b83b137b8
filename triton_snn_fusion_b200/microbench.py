"""Single-kernel timing of the library's fused ops through the C ABI.

    python -m triton_snn_fusion_b200.microbench conv --B 64 --cin 128 --cout 128 --hw 56
    python -m triton_snn_fusion_b200.microbench lif  --n 16777216
    python -m triton_snn_fusion_b200.microbench dw   --B 32 --c 128 --hw 56
    python -m triton_snn_fusion_b200.microbench tail --B 256 --c 1024 --hw 7 --classes 1000
    python -m triton_snn_fusion_b200.microbench stem --B 128 --hw 224
    python -m triton_snn_fusion_b200.microbench linear --M 4096 --K 768 --N 3072
    python -m triton_snn_fusion_b200.microbench mma                # cycles per tcgen05.mma for M x N shapes

Each case builds seeded synthetic spikes/currents on the GPU (larger than L2 at the default sizes),
warms the op up three times, times `--reps` launches with CUDA events and prints the algorithmic
GB/s and TFLOP/s. With `--reps 1` it is the small case a profiler is pointed at.

The conv case follows the workload of the reference's conv + LIF kernel benchmark
(benchmarks/benchmark_fused_convlif_kernel_configs.py: conv + folded BN + LIF over T steps).
"""
from __future__ import annotations

import argparse

import torch

from . import _lib

DEV = "cuda"
LIF = (1.0, 0.0, 2.0)   # v_th, v_reset, tau: the reference's defaults


def _time(call, reps):
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        call()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def _stream():
    return torch.cuda.current_stream().cuda_stream


def case_conv(a):
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float16
    p = (a.k - 1) // 2
    ho = (a.hw + 2 * p - a.k) // a.s + 1
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.rand(a.T, a.B, a.hw, a.hw, a.cin, device=DEV, generator=g) < 0.15).to(dt)
    w = (torch.randn(a.cout, a.k, a.k, a.cin, device=DEV, generator=g)
         * (2.0 / (a.cin * a.k * a.k)) ** 0.5 * 2.5).to(dt)
    b = (torch.randn(a.cout, device=DEV, generator=g) * 0.1).to(dt)
    res = (torch.rand(a.T, a.B, ho, ho, a.cout, device=DEV, generator=g) < 0.2).to(dt) if a.res else None
    sp = torch.empty(a.T, a.B, ho, ho, a.cout, device=DEV, dtype=dt)
    v = torch.empty(a.B, ho, ho, a.cout, device=DEV, dtype=dt)
    dc = _lib.dtype_code(dt)

    def call():
        st = _lib.lib.snnb_conv_lif(
            x.data_ptr(), x.stride(0), w.data_ptr(), b.data_ptr(),
            res.data_ptr() if res is not None else None, None, sp.data_ptr(), v.data_ptr(),
            a.T, a.B, a.cin, a.hw, a.hw, a.cout, a.k, a.k, a.s, p,
            1, dc, dc, dc, *LIF, a.path, _stream())
        _lib.check(st, "snnb_conv_lif")

    ms = _time(call, a.reps)
    flops = 2.0 * a.T * a.B * ho * ho * a.cout * a.cin * a.k * a.k
    nbytes = 2 * (x.numel() + sp.numel() + v.numel() + w.numel() + (res.numel() if res is not None else 0))
    print(f"conv_lif B{a.B} {a.cin}->{a.cout} k{a.k}s{a.s} {a.hw}^2 T{a.T} res={a.res} path={a.path}: "
          f"{ms:.4f} ms  {flops / ms / 1e9:.1f} TFLOP/s  {nbytes / ms / 1e6:.0f} GB/s  "
          f"spike rate {float(sp.float().mean()):.3f}  device status {_lib.device_status()}")


def case_lif(a):
    dt = {"f32": torch.float32, "bf16": torch.bfloat16}[a.dtype]
    dc = _lib.dtype_code(dt)
    es = 4 if a.dtype == "f32" else 2
    # Footprints below the L2 size would be served from L2 on every repetition: rotate through enough copies of the
    # buffers that a launch never finds its data cached (every copy holds different seeded values).
    footprint = es * (2 * a.T + 1) * a.n
    copies = max(1, -(-(400 << 20) // footprint)) if footprint < (256 << 20) else 1
    g = torch.Generator(device=DEV).manual_seed(0)
    xs = [(torch.randn(a.T, a.n, device=DEV, generator=g) * 0.8 + 0.6).to(dt) for _ in range(copies)]
    sps = [torch.empty_like(x) for x in xs]
    vs = [torch.empty(a.n, device=DEV, dtype=dt) for _ in range(copies)]
    k = [0]

    def call():
        i = k[0] % copies
        k[0] += 1
        _lib.check(_lib.lib.snnb_lif_scan(xs[i].data_ptr(), None, sps[i].data_ptr(), vs[i].data_ptr(), a.T, a.n,
                                          dc, dc, dc, *LIF, _stream()), "snnb_lif_scan")

    ms = _time(call, max(a.reps, 2 * copies))
    print(f"lif_scan T{a.T} n={a.n} {a.dtype}: {ms:.4f} ms  {footprint / ms / 1e6:.0f} GB/s  "
          f"spike rate {float(sps[0].float().mean()):.3f}  ({copies} rotating buffer sets)")


def case_dw(a):
    dt = torch.bfloat16
    ho = (a.hw - 1) // a.s + 1
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.rand(a.T, a.B, a.hw, a.hw, a.c, device=DEV, generator=g) < 0.2).to(dt)
    w = (torch.randn(a.c, 3, 3, device=DEV, generator=g) * 0.3).to(dt)
    b = torch.zeros(a.c, device=DEV, dtype=dt)
    sp = torch.empty(a.T, a.B, ho, ho, a.c, device=DEV, dtype=dt)
    v = torch.empty(a.B, ho, ho, a.c, device=DEV, dtype=dt)

    def call():
        _lib.check(_lib.lib.snnb_dwconv3x3_lif(x.data_ptr(), x.stride(0), w.data_ptr(), b.data_ptr(), None, None,
                                               sp.data_ptr(), v.data_ptr(), a.T, a.B, a.c, a.hw, a.hw, a.s,
                                               1, 1, 1, *LIF, _stream()), "snnb_dwconv3x3_lif")

    ms = _time(call, a.reps)
    nbytes = 2 * (x.numel() + sp.numel() + v.numel())
    print(f"dwconv3x3_lif B{a.B} C{a.c} {a.hw}^2 s{a.s} T{a.T} bf16: {ms:.4f} ms  {nbytes / ms / 1e6:.0f} GB/s  "
          f"spike rate {float(sp.float().mean()):.3f}  device status {_lib.device_status()}")


def case_tail(a):
    dt = torch.bfloat16
    hw = a.hw * a.hw
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.randn(a.T, a.B, hw, a.c, device=DEV, generator=g) * 0.75 + 0.15).to(dt)
    w = (torch.randn(a.classes, a.c, device=DEV, generator=g) * 0.05).to(dt)
    b = torch.zeros(a.classes, device=DEV, dtype=dt)
    out = torch.empty(a.B, a.classes, device=DEV, dtype=dt)
    v = torch.empty(a.B, hw, a.c, device=DEV, dtype=dt)

    def call():
        _lib.check(_lib.lib.snnb_lif_avgpool_linear(x.data_ptr(), None, w.data_ptr(), b.data_ptr(), out.data_ptr(),
                                                    v.data_ptr(), a.T, a.B, a.c, hw, a.classes, 1, 1, 1,
                                                    *LIF, _stream()), "snnb_lif_avgpool_linear")

    ms = _time(call, a.reps)
    nbytes = 2 * (x.numel() + v.numel() + w.numel() + out.numel())
    print(f"lif_avgpool_linear B{a.B} C{a.c} {a.hw}^2 -> {a.classes} T{a.T} bf16: {ms:.4f} ms  "
          f"{nbytes / ms / 1e6:.0f} GB/s")


def case_linear(a):
    dt = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(0)
    if a.dist == "normal":   # real-valued activations N(0, 1), weights N(0, 1 / sqrt(K))
        x = torch.randn(a.T, a.M, a.K, device=DEV, generator=g).to(dt)
        w = (torch.randn(a.N, a.K, device=DEV, generator=g) * a.K ** -0.5).to(dt)
    else:                    # binary spikes Bernoulli(0.15), as a preceding LIF layer would emit
        x = (torch.rand(a.T, a.M, a.K, device=DEV, generator=g) < 0.15).to(dt)
        w = (torch.randn(a.N, a.K, device=DEV, generator=g) * a.K ** -0.5 * 2.5).to(dt)
    b = torch.zeros(a.N, device=DEV, dtype=dt)
    sp = torch.empty(a.T, a.M, a.N, device=DEV, dtype=dt)
    v = torch.empty(a.M, a.N, device=DEV, dtype=dt)

    def call():
        _lib.check(_lib.lib.snnb_linear_lif(x.data_ptr(), x.stride(0), w.data_ptr(), b.data_ptr(), None, sp.data_ptr(),
                                            v.data_ptr(), a.T, a.M, a.K, a.N, 1, 1, 1, *LIF, a.path, _stream()),
                   "snnb_linear_lif")

    ms = _time(call, a.reps)
    flops = 2.0 * a.T * a.M * a.K * a.N
    nbytes = 2 * (x.numel() + sp.numel() + v.numel() + w.numel())
    print(f"linear_lif T{a.T} M{a.M} K{a.K} N{a.N} bf16 ({a.dist} inputs): {ms:.4f} ms  {flops / ms / 1e9:.1f} TFLOP/s  "
          f"{nbytes / ms / 1e6:.0f} GB/s  spike rate {float(sp.float().mean()):.3f}  device status {_lib.device_status()}")


def case_stem(a):
    dt = torch.bfloat16
    ho = a.hw // 2
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(a.B, a.hw, a.hw, 3, device=DEV, generator=g).to(dt)
    w = (torch.randn(a.cout, 7, 7, 3, device=DEV, generator=g) * (2.0 / 147) ** 0.5).to(dt)
    b = (torch.randn(a.cout, device=DEV, generator=g) * 0.1).to(dt)
    wp = torch.empty(a.cout, 256, device=DEV, dtype=dt)
    _lib.check(_lib.lib.snnb_stem7x7_pack_weight(w.data_ptr(), wp.data_ptr(), a.cout, 1, _stream()), "pack")
    nscratch = int(_lib.lib.snnb_stem7x7_scratch_bytes(a.B, a.hw, a.hw))
    scratch = torch.empty(nscratch, device=DEV, dtype=torch.uint8)
    # spikes in the activation dtype with a membrane output (the drop-in form), or one byte / one bit each without
    # one (the executor's form)
    if a.spikes == "same":
        sp = torch.empty(a.T, a.B, ho, ho, a.cout, device=DEV, dtype=dt)
        v, sdt = torch.empty(a.B, ho, ho, a.cout, device=DEV, dtype=dt), 1
    elif a.spikes == "u8":
        sp, v, sdt = torch.empty(a.T, a.B, ho, ho, a.cout, device=DEV, dtype=torch.uint8), None, _lib.U8
    else:
        sp, v, sdt = torch.empty(a.T, a.B, ho, ho, a.cout // 8, device=DEV, dtype=torch.uint8), None, _lib.B1

    def call():   # one frame for all T steps (direct encoding)
        _lib.check(_lib.lib.snnb_stem7x7_lif(x.data_ptr(), 0, wp.data_ptr(), b.data_ptr(), None, sp.data_ptr(),
                                             v.data_ptr() if v is not None else None, scratch.data_ptr(), nscratch,
                                             a.T, a.B, a.hw, a.hw, a.cout, 1, sdt, 1, *LIF, _stream()), "snnb_stem7x7_lif")

    ms = _time(call, a.reps)
    nbytes = 2 * x.numel() + sp.numel() * sp.element_size() + (2 * v.numel() if v is not None else 0) + 2 * nscratch
    rate = float(sp.float().mean()) if a.spikes != "bits" else float("nan")
    print(f"stem7x7_lif B{a.B} 3->{a.cout} {a.hw}^2 T{a.T} bf16, spikes {a.spikes} (s2d + GEMM): {ms:.4f} ms  "
          f"{nbytes / ms / 1e6:.0f} GB/s  spike rate {rate:.3f}  device status {_lib.device_status()}")


def case_mma(a):
    """SM cycles per tcgen05.mma (K = 16, bf16, fp32 accumulate) for the shapes the tile layouts choose between,
    with one block on the GPU and with one block on every SM; then the 128 x 256 shape on every SM for about 0.2 s
    with zero and with random operands: cycles per instruction and the SM clock the blocks really ran at."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def probe(M, N, reps, ctas, fill, commit_every=0, nslots=1):
        cyc = torch.zeros(ctas, dtype=torch.int64, device=DEV)
        ns = torch.zeros(ctas, dtype=torch.int64, device=DEV)
        st = torch.zeros(1, dtype=torch.int32, device=DEV)
        for _ in range(2):   # the first launch also pays for set-up
            _lib.check(_lib.lib.snnb_probe_mma_cycles(M, N, reps, ctas, fill, commit_every, nslots, cyc.data_ptr(), ns.data_ptr(), st.data_ptr(), None), "probe")
        torch.cuda.synchronize()
        if int(st.item()) != 0 or int(cyc.min().item()) < 0:
            raise SystemExit(f"probe M={M} N={N}: a bounded wait gave up")
        return cyc.double(), ns.double()

    print(f"cycles per tcgen05.mma.kind::f16 M x N x 16 ({4 * a.reps_mma} instructions behind one commit); "
          f"128 x 256 x 16 at the nominal dense rate is 128 cycles")
    print(f"{'M':>4} {'N':>4}  {'1 block':>9}  {'%d blocks (mean / max)' % sms:>24}  useful MACs per cycle and SM (all blocks)")
    for M in (128, 64):
        for N in (64, 128, 256):
            one, _ = probe(M, N, a.reps_mma, 1, 0)
            allc, _ = probe(M, N, a.reps_mma, sms, 0)
            per1, per = one / (4 * a.reps_mma), allc / (4 * a.reps_mma)
            print(f"{M:>4} {N:>4}  {float(per1.mean()):9.1f}  {float(per.mean()):11.1f} / {float(per.max()):<10.1f}  "
                  f"{M * N * 16 / float(per.mean()):8.0f}")
    for ce in (1, 2, 4):
        c, _ = probe(128, 256, a.reps_mma, sms, 0, ce)
        print(f" 128  256  with a tcgen05.commit after every {ce} batch(es) of four: {float(c.mean()) / (4 * a.reps_mma):7.1f} cycles per instruction")
    for ns in (2, 4):
        for N in (128, 256):
            c, _ = probe(128, N, a.reps_mma, sms, 1, 1, ns)
            print(f" 128 {N:4d}  batches cycling through {ns} operand tile pairs (random values, commit per batch): "
                  f"{float(c.mean()) / (4 * a.reps_mma):7.1f} cycles per instruction")
    long_reps = 1 << 18   # 2^20 instructions of 128 cycles: about 0.07 s at full clock
    print(f"128 x 256 x 16 on {sms} blocks, {4 * long_reps} instructions each:")
    for fill, name in ((0, "zero operands"), (1, "random operands")):
        cyc, ns = probe(128, 256, long_reps, sms, fill)
        mhz = float((cyc / ns).mean()) * 1e3
        tflops = sms * 2 * 128 * 256 * 16 * 4 * long_reps / float(ns.mean()) * 1e9 / 1e12
        print(f"  {name:16s} {float(cyc.mean()) / (4 * long_reps):7.1f} cycles per instruction, SM clock {mhz:6.0f} MHz, {tflops:7.1f} TFLOP/s")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="case", required=True)
    c = sub.add_parser("conv")
    c.add_argument("--B", type=int, default=64)
    c.add_argument("--cin", type=int, default=128)
    c.add_argument("--cout", type=int, default=128)
    c.add_argument("--hw", type=int, default=56)
    c.add_argument("--k", type=int, default=3)
    c.add_argument("--s", type=int, default=1)
    c.add_argument("--res", type=int, default=0)
    c.add_argument("--dtype", choices=["bf16", "f16"], default="bf16")
    c.add_argument("--path", type=int, default=_lib.PATH_TCGEN05,
                   help="snnb_path: 0 auto, 1 simt, 2 tcgen05, 3 per-tap kernel, 4 halo kernel")
    c.set_defaults(fn=case_conv)
    l = sub.add_parser("lif")
    l.add_argument("--n", type=int, default=1 << 24)
    l.add_argument("--dtype", choices=["f32", "bf16"], default="f32")
    l.set_defaults(fn=case_lif)
    d = sub.add_parser("dw")
    d.add_argument("--B", type=int, default=32)
    d.add_argument("--c", type=int, default=128)
    d.add_argument("--hw", type=int, default=56)
    d.add_argument("--s", type=int, default=1)
    d.set_defaults(fn=case_dw)
    t = sub.add_parser("tail")
    t.add_argument("--B", type=int, default=256)
    t.add_argument("--c", type=int, default=1024)
    t.add_argument("--hw", type=int, default=7)
    t.add_argument("--classes", type=int, default=1000)
    t.set_defaults(fn=case_tail)
    m = sub.add_parser("stem")
    m.add_argument("--B", type=int, default=128)
    m.add_argument("--hw", type=int, default=224)
    m.add_argument("--cout", type=int, default=64)
    m.add_argument("--spikes", choices=["same", "u8", "bits"], default="same")
    m.set_defaults(fn=case_stem)
    n = sub.add_parser("linear")
    n.add_argument("--M", type=int, default=4096)
    n.add_argument("--K", type=int, default=768)
    n.add_argument("--N", type=int, default=3072)
    n.add_argument("--path", type=int, default=_lib.PATH_TCGEN05)
    n.add_argument("--dist", choices=["bernoulli", "normal"], default="bernoulli")
    n.set_defaults(fn=case_linear)
    q = sub.add_parser("mma")
    q.add_argument("--reps-mma", type=int, default=512, help="batches of four MMAs per measurement")
    q.set_defaults(fn=case_mma)
    for p in (c, l, d, t, m, n):
        p.add_argument("--T", type=int, default=4)
        p.add_argument("--reps", type=int, default=10)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    a.fn(a)


if __name__ == "__main__":
    main()
