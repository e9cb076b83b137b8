"""Whole networks on the fused kernels against the oracle, layer by layer.

Each layer of the device run is compared with the oracle evaluated on the DEVICE's inputs to that
layer ("teacher forcing"), so the flip-rate / membrane bounds are per layer and a flip in one layer
does not leak into the verdict on the next. End-to-end logits are compared as well.
"""
import pytest
import torch

from oracle import models as omodels
from util import check_parity

pytestmark = pytest.mark.gpu


def _run_net(name, B, T, hw, dtype, classes, path="auto"):
    from triton_snn_fusion_b200 import nets
    spec = nets.NETS[name](classes)
    params = nets.make_params(spec, seed=2026)
    net = nets.CompiledNet(spec, params, batch=B, T=T, in_hw=(hw, hw), dtype=dtype, device="cuda", conv_path=path,
                           keep_membranes=True)
    x = torch.randn(B, 3, hw, hw, generator=torch.Generator().manual_seed(2026)).to(dtype)
    logits = net.forward_nchw(x.cuda()).cpu()
    torch.cuda.synchronize()
    teacher = {n: net.activation(n).cpu() for n in net.bufs if n != "input"}
    folded = nets.folded_params(spec, params, dtype)
    ref_logits, layers = omodels.folded_forward(spec, folded, x, T, teacher=teacher)
    return spec, net, logits, teacher, ref_logits, layers


def _check_layers(spec, net, teacher, layers, dtype):
    worst = 0.0
    for L in spec:
        if L["op"] == "conv" and L["lif"]:
            v = net.membranes[L["name"]].permute(0, 3, 1, 2).cpu()
            rate = check_parity(teacher[L["dst"]], v, layers[L["name"]][0], layers[L["name"]][1], dtype,
                                flip_max=2e-4, what=L["name"])
            worst = max(worst, rate)
        elif L["op"] == "conv":
            rtol, atol = (1e-4, 1e-5) if dtype == torch.float32 else (1e-2, 1e-2)
            torch.testing.assert_close(teacher[L["dst"]].float(), layers[L["name"]][0], rtol=rtol, atol=atol)
        elif L["op"] == "maxpool":
            assert torch.equal(teacher[L["dst"]].float(), layers[L["name"]][0])
    return worst


def test_cnn_small_fp32_config0():
    """BASELINE config 0: CNN-small, fp32, T=4, batch 16, 3x32x32."""
    spec, net, logits, teacher, ref_logits, layers = _run_net("cnn_small", 16, 4, 32, torch.float32, 10)
    _check_layers(spec, net, teacher, layers, torch.float32)
    torch.testing.assert_close(logits, ref_logits, rtol=1e-4, atol=1e-4)
    # un-fused eager model with un-folded BatchNorm gives the same logits
    from triton_snn_fusion_b200 import nets
    eager = omodels.eager_forward(spec, nets.make_params(spec, seed=2026),
                                  torch.randn(16, 3, 32, 32, generator=torch.Generator().manual_seed(2026)), 4)
    torch.testing.assert_close(logits, eager, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_resnet18_small_input(dtype):
    spec, net, logits, teacher, ref_logits, layers = _run_net("resnet18", 2, 4, 64, dtype, 100)
    _check_layers(spec, net, teacher, layers, dtype)
    tol = 1e-3 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(logits, ref_logits, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mobilenet_v1_small_input(dtype):
    spec, net, logits, teacher, ref_logits, layers = _run_net("mobilenet_v1", 2, 4, 64, dtype, 100)
    _check_layers(spec, net, teacher, layers, dtype)
    tol = 1e-3 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(logits, ref_logits, rtol=tol, atol=tol)


def test_cuda_graph_replay_matches_eager_issue():
    from triton_snn_fusion_b200 import nets
    spec = nets.spiking_resnet18(100)
    params = nets.make_params(spec, seed=5)
    net = nets.CompiledNet(spec, params, batch=2, T=4, in_hw=(64, 64), dtype=torch.bfloat16, device="cuda")
    x = torch.randn(2, 64, 64, 3, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    a = net.forward(x).clone()
    net.capture()
    b = net.forward(x).clone()
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("name,dtype", [("resnet18", torch.bfloat16), ("resnet18", torch.float32),
                                        ("mobilenet_v1", torch.bfloat16)])
def test_forward_without_membrane_outputs(name, dtype):
    """v_out = NULL (the executor's default): same spikes, hence bit-identical logits."""
    from triton_snn_fusion_b200 import nets
    spec = nets.NETS[name](100)
    params = nets.make_params(spec, seed=7)
    x = torch.randn(2, 64, 64, 3, generator=torch.Generator().manual_seed(3)).to(dtype).cuda()
    outs = []
    for keep in (True, False):
        net = nets.CompiledNet(spec, params, batch=2, T=4, in_hw=(64, 64), dtype=dtype, device="cuda",
                               keep_membranes=keep)
        outs.append(net.forward(x).clone())
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])


def test_pipelined_submit_matches_forward():
    """submit(): staged host->device copies on a side stream; same logits as forward() for every batch."""
    from triton_snn_fusion_b200 import nets
    spec = nets.spiking_resnet18(100)
    params = nets.make_params(spec, seed=5)
    net = nets.CompiledNet(spec, params, batch=2, T=4, in_hw=(64, 64), dtype=torch.bfloat16, device="cuda")
    g = torch.Generator().manual_seed(11)
    batches = [torch.randn(2, 64, 64, 3, generator=g).to(torch.bfloat16).pin_memory() for _ in range(5)]
    want = []
    for b in batches:
        want.append(net.forward(b.cuda()).clone())
    net.capture()
    outs = [torch.empty(2, 100, dtype=torch.float32).pin_memory() for _ in batches]
    for b, o in zip(batches, outs):
        net.submit(b, o)
    torch.cuda.synchronize()
    for w, o in zip(want, outs):
        assert torch.equal(w.cpu(), o)
