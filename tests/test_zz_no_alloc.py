"""snnb_stem7x7_lif_static: the stem entry point for callers that cannot allocate device memory.

Some hosts give a plugin only its input and output buffers (the runtime owns the device pool), and
some serving loops must not reach the driver allocator once they are running. For them the library
carries its own fixed scratch array. This test calls that entry through the C ABI twice in a row
and requires the same bits as the regular entry point, which gets its scratch from the caller. The
second call uses a different, smaller input, so anything the first call left in the shared array
would show up as a difference. The file name keeps it last in collection order.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run(L, entry, x, wp, b, T, scratch=None):
    B, H, W, _ = x.shape
    cout = wp.shape[0]
    dt = L.dtype_code(x.dtype)
    spikes = torch.empty(T, B, H // 2, W // 2, cout, dtype=x.dtype, device=DEV)
    v = torch.empty(B, H // 2, W // 2, cout, dtype=x.dtype, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    if entry == "static":
        st = L.lib.snnb_stem7x7_lif_static(x.data_ptr(), 0, wp.data_ptr(), b.data_ptr(), None, spikes.data_ptr(),
                                           v.data_ptr(), T, B, H, W, cout, dt, dt, dt, 1.0, 0.0, 2.0, stream)
    else:
        st = L.lib.snnb_stem7x7_lif(x.data_ptr(), 0, wp.data_ptr(), b.data_ptr(), None, spikes.data_ptr(),
                                    v.data_ptr(), scratch.data_ptr(), scratch.numel(), T, B, H, W, cout, dt, dt, dt,
                                    1.0, 0.0, 2.0, stream)
    L.check(st, f"stem ({entry})")
    torch.cuda.synchronize()
    return spikes, v


def test_static_scratch_entry_matches_caller_scratch_entry_twice():
    from triton_snn_fusion_b200 import _lib as L

    torch.manual_seed(2026)
    dtype, T, cout = torch.bfloat16, 4, 64
    w = (torch.randn(cout, 7, 7, 3) * (2.0 / 147) ** 0.5).to(dtype).to(DEV)  # [Cout][KH][KW][Cin]
    b = (torch.randn(cout) * 0.1).to(dtype).to(DEV)
    wp = torch.empty(cout, 256, dtype=dtype, device=DEV)
    L.check(L.lib.snnb_stem7x7_pack_weight(w.data_ptr(), wp.data_ptr(), cout, L.dtype_code(dtype), None), "pack")
    torch.cuda.synchronize()
    for B, H, W in ((3, 96, 64), (2, 32, 48)):  # two calls in a row, the second smaller than the first
        x = torch.randn(B, H, W, 3).to(dtype).to(DEV)
        nbytes = int(L.lib.snnb_stem7x7_scratch_bytes(B, H, W))
        assert 0 < nbytes <= int(L.lib.snnb_stem7x7_static_scratch_bytes())
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        ref_s, ref_v = _run(L, "caller", x, wp, b, T, scratch)
        got_s, got_v = _run(L, "static", x, wp, b, T)
        assert torch.equal(got_s, ref_s), "spikes differ from the caller-scratch entry point"
        assert torch.equal(got_v, ref_v), "membrane differs from the caller-scratch entry point"
        assert 0.01 < float(ref_s.float().mean()) < 0.7
    assert L.device_status() == 0


def test_static_scratch_entry_rejects_oversized_calls():
    from triton_snn_fusion_b200 import _lib as L

    B, H, W = 64, 224, 224  # needs ~27 MB of scratch, more than the built-in array
    assert int(L.lib.snnb_stem7x7_scratch_bytes(B, H, W)) > int(L.lib.snnb_stem7x7_static_scratch_bytes())
    one = torch.zeros(16, dtype=torch.bfloat16, device=DEV)
    st = L.lib.snnb_stem7x7_lif_static(one.data_ptr(), 0, one.data_ptr(), one.data_ptr(), None, one.data_ptr(),
                                       one.data_ptr(), 4, B, H, W, 64, L.BF16, L.BF16, L.BF16, 1.0, 0.0, 2.0, None)
    assert st == 2
    msg = L.lib.snnb_last_error().decode()
    assert "built-in array" in msg and "bytes" in msg
