"""Stateless channels-last helpers against torch on the CPU."""
import time

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lib():
    from triton_snn_fusion_b200 import _lib
    return _lib


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 3, 7, 9), (2, 64, 14, 14), (1, 33, 1, 1)])
def test_layout_round_trip(dtype, shape):
    L = _lib()
    F_, C, H, W = shape
    x = torch.randn(shape).to(dtype)
    xd = x.to(DEV)
    y = torch.empty(F_, H, W, C, dtype=dtype, device=DEV)
    L.check(L.lib.snnb_nchw_to_nhwc(xd.data_ptr(), y.data_ptr(), F_, C, H * W, L.dtype_code(dtype), None), "t")
    assert torch.equal(y.cpu(), x.permute(0, 2, 3, 1).contiguous())
    back = torch.empty_like(xd)
    L.check(L.lib.snnb_nhwc_to_nchw(y.data_ptr(), back.data_ptr(), F_, C, H * W, L.dtype_code(dtype), None), "t")
    assert torch.equal(back.cpu(), x)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(3, 64, 16, 16), (2, 6, 9, 7), (1, 8, 112, 112)])
def test_maxpool(dtype, shape):
    L = _lib()
    F_, C, H, W = shape
    x = (torch.rand(shape) < 0.3).to(dtype)
    ref = F.max_pool2d(x.float(), 3, 2, 1)
    xd = x.permute(0, 2, 3, 1).contiguous().to(DEV)
    Ho, Wo = ref.shape[2], ref.shape[3]
    y = torch.empty(F_, Ho, Wo, C, dtype=dtype, device=DEV)
    L.check(L.lib.snnb_maxpool3x3s2(xd.data_ptr(), y.data_ptr(), F_, H, W, C, L.dtype_code(dtype), None), "maxpool")
    assert torch.equal(y.cpu().float().permute(0, 3, 1, 2), ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(3, 64, 16, 16), (2, 16, 9, 7), (1, 32, 112, 112)])
def test_maxpool_of_byte_spikes(dtype, shape):
    """snnb_maxpool3x3s2_u8: one-byte spikes in, pooled spikes in the activation dtype out."""
    L = _lib()
    F_, C, H, W = shape
    x = (torch.rand(shape) < 0.3)
    ref = F.max_pool2d(x.float(), 3, 2, 1)
    xd = x.to(torch.uint8).permute(0, 2, 3, 1).contiguous().to(DEV)
    Ho, Wo = ref.shape[2], ref.shape[3]
    y = torch.empty(F_, Ho, Wo, C, dtype=dtype, device=DEV)
    L.check(L.lib.snnb_maxpool3x3s2_u8(xd.data_ptr(), y.data_ptr(), F_, H, W, C, L.dtype_code(dtype), None), "maxpool_u8")
    assert torch.equal(y.cpu().float().permute(0, 3, 1, 2), ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_avgpool_linear_mean(dtype):
    L = _lib()
    T, N, C, H, W, K = 4, 6, 512, 7, 7, 1000
    torch.manual_seed(0)
    x = (torch.rand(T, N, C, H, W) < 0.2).to(dtype)
    w = (torch.randn(K, C) * 0.05).to(dtype)
    b = (torch.randn(K) * 0.05).to(dtype)
    ref = torch.stack([F.linear(F.adaptive_avg_pool2d(x[t].float(), 1).flatten(1), w.float(), b.float())
                       for t in range(T)]).mean(0)
    xd = x.permute(0, 1, 3, 4, 2).contiguous().to(DEV)
    out = torch.empty(N, K, device=DEV)
    wd, bd = w.to(DEV), b.to(DEV)  # keep the device copies alive across the call
    L.check(L.lib.snnb_avgpool_linear_mean(xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), out.data_ptr(),
                                           T, N, C, H * W, K, L.dtype_code(dtype), None), "head")
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("N", [3, 64, 301])
def test_avgpool_linear_mean_arbitrary_values(N):
    """bf16 inputs that are not spikes: the tensor-core form keeps each pooled sum as two bf16 parts."""
    L = _lib()
    T, C, HW, K = 4, 512, 49, 1000
    torch.manual_seed(N)
    x = (torch.randn(T, N, HW, C) * 0.7 + 0.2).to(torch.bfloat16)
    w = (torch.randn(K, C) * 0.05).to(torch.bfloat16)
    b = (torch.randn(K) * 0.05).to(torch.bfloat16)
    ref = x.float().mean(dim=(0, 2)) @ w.float().t() + b.float()
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    out = torch.empty(N, K, device=DEV)
    L.check(L.lib.snnb_avgpool_linear_mean(xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), out.data_ptr(),
                                           T, N, C, HW, K, L.BF16, None), "head")
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-3, atol=1e-4)
    out2 = torch.empty_like(out)
    L.check(L.lib.snnb_avgpool_linear_mean(xd.data_ptr(), wd.data_ptr(), bd.data_ptr(), out2.data_ptr(),
                                           T, N, C, HW, K, L.BF16, None), "head")
    assert torch.equal(out, out2)   # fixed summation order


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_reports():
    """A wait inside the tcgen05 conv kernel that can never complete (a weight tile that is announced but not
    loaded, limit shortened to about a millisecond) must end by itself: the call returns, the status word says
    that a wait gave up, and the next call works and leaves the status clean."""
    from oracle import snn_oracle as orc
    from triton_snn_fusion_b200 import _lib as L
    from util import check_parity
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(1)
    x = (torch.rand(4, 2, 16, 16, 64, generator=g) < 0.2).to(dtype)
    w = (torch.randn(128, 3, 3, 64, generator=g) * 0.12).to(dtype)
    b = (torch.randn(128, generator=g) * 0.1).to(dtype)
    xd, wd, bd = x.cuda(), w.cuda(), b.cuda()
    spikes = torch.zeros(4, 2, 16, 16, 128, dtype=dtype, device="cuda")
    v = torch.zeros(2, 16, 16, 128, dtype=dtype, device="cuda")

    def call():
        L.check(L.lib.snnb_conv_lif(xd.data_ptr(), xd.stride(0), wd.data_ptr(), bd.data_ptr(), None, None,
                                    spikes.data_ptr(), v.data_ptr(), 4, 2, 64, 16, 16, 128, 3, 3, 1, 1, 1,
                                    L.BF16, L.BF16, L.BF16, 1.0, 0.0, 2.0, L.PATH_TCGEN05, None), "snnb_conv_lif")
        torch.cuda.synchronize()

    assert L.device_status() == 0
    L.check(L.lib.snnb_selftest_arm_wait_timeout(2_000_000), "arm")
    t0 = time.perf_counter()
    call()
    assert time.perf_counter() - t0 < 5.0
    assert L.device_status() != 0        # reported once ...
    assert L.device_status() == 0        # ... and cleared by the read
    call()                               # the hook disarmed itself: a normal run
    assert L.device_status() == 0
    rs, rv = orc.temporal_conv_lif([orc.widen(x[t]).permute(0, 3, 1, 2) for t in range(4)],
                                   orc.widen(w).permute(0, 3, 1, 2), orc.widen(b), None, [1, 1], [1, 1], [1, 1], 1,
                                   1.0, 0.0, 2.0)
    check_parity(spikes.permute(0, 1, 4, 2, 3), v.permute(0, 3, 1, 2), rs, rv, dtype, what="after the self-test")


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(5, 14, 18, 64), (2, 7, 9, 128), (3, 112, 112, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_maxpool_of_bit_packed_spikes(shape, dtype):
    """snnb_maxpool3x3s2_bits (spikes one bit each, 32 channels per word) against torch's max_pool2d."""
    L = _lib()
    frames, H, W, C = shape
    g = torch.Generator().manual_seed(H * W + C)
    spikes = (torch.rand(frames, H, W, C, generator=g) < 0.2)
    weights = (1 << torch.arange(8, dtype=torch.int32)).to(torch.uint8)
    packed = (spikes.reshape(frames, H, W, C // 8, 8).to(torch.uint8) * weights).sum(-1).to(torch.uint8).contiguous()
    Ho, Wo = (H - 1) // 2 + 1, (W - 1) // 2 + 1
    y = torch.empty(frames, Ho, Wo, C, dtype=dtype, device=DEV)
    xd = packed.to(DEV)
    L.check(L.lib.snnb_maxpool3x3s2_bits(xd.data_ptr(), y.data_ptr(), frames, H, W, C, L.dtype_code(dtype), None), "pool bits")
    want = F.max_pool2d(spikes.float().permute(0, 3, 1, 2), 3, 2, 1).permute(0, 2, 3, 1)
    assert torch.equal(y.float().cpu(), want)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N", [(128, 256), (128, 64), (64, 128)])
def test_mma_probe_reports_cycles(M, N):
    """The tcgen05.mma timing probe ends by itself and reports a positive cycle count for every block."""
    L = _lib()
    ctas, reps = 6, 32
    cyc = torch.zeros(ctas, dtype=torch.int64, device=DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    ns = torch.zeros(ctas, dtype=torch.int64, device=DEV)
    L.check(L.lib.snnb_probe_mma_cycles(M, N, reps, ctas, 1, 1, 3, cyc.data_ptr(), ns.data_ptr(), st.data_ptr(), None), "probe")
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert bool((cyc > 0).all()) and bool((ns > 0).all())
    per = float(cyc.double().mean()) / (4 * reps)
    assert 8.0 < per < 5000.0, per
    with pytest.raises(L.SnnbError):
        L.check(L.lib.snnb_probe_mma_cycles(96, N, reps, ctas, 0, 0, 1, cyc.data_ptr(), None, st.data_ptr(), None), "probe")
