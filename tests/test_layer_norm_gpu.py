"""Row normalisation kernels (grws_layer_norm_fwd / _bwd) against torch's fp32 LayerNorm of the same
rounded operands."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,C", [(1, 16), (37, 128), (5000, 256), (333, 264), (129, 1024), (0, 64)])
def test_forward_and_backward_match_torch(rows, C, dtype, relu):
    from graph_rws_b200.layers.norm import act_layer_norm
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(rows * 131 + C)
    x = torch.randn(rows, C, generator=g).to(dtype).to(dev).requires_grad_(True)
    norm = torch.nn.LayerNorm(C).to(dev)
    with torch.no_grad():
        norm.weight.copy_(1.0 + 0.3 * torch.randn(C, generator=g))
        norm.bias.copy_(0.2 * torch.randn(C, generator=g))
    norm = norm.to(dtype)
    dy = torch.randn(rows, C, generator=g).to(dtype).to(dev)
    y = act_layer_norm(x, norm, relu)
    assert y.dtype == dtype and y.shape == (rows, C)
    y.backward(dy)
    got = (y.detach().float(), x.grad.float(), norm.weight.grad.float(), norm.bias.grad.float())
    # fp32 reference on the same rounded operands
    x32 = x.detach().float().requires_grad_(True)
    w32 = norm.weight.detach().float().requires_grad_(True)
    b32 = norm.bias.detach().float().requires_grad_(True)
    y32 = F.layer_norm(F.relu(x32) if relu else x32, (C,), w32, b32, norm.eps)
    y32.backward(dy.float())
    want = (y32.detach(), x32.grad, w32.grad, b32.grad)
    tol = TOL[dtype]
    for name, a, b in zip(("y", "dx", "dgamma", "dbeta"), got, want):
        scale = max(float(b.abs().max()) if b.numel() else 0.0, 1.0)
        # parameter gradients are sums over the rows, rounded once to the parameter dtype
        assert float((a - b).abs().max()) <= tol * scale if a.numel() else True, name


def test_model_uses_the_kernels_and_unsupported_shapes_fall_back():
    from graph_rws_b200.layers.norm import act_layer_norm
    dev = torch.device("cuda")
    x = torch.randn(50, 20, device=dev)                  # 20 is no multiple of 8: torch's operators
    norm = torch.nn.LayerNorm(20).to(dev)
    torch.testing.assert_close(act_layer_norm(x, norm, True), norm(F.relu(x)))
    x = torch.randn(64, 64, device=dev)
    norm = torch.nn.LayerNorm(64).to(dev)
    torch.testing.assert_close(act_layer_norm(x, norm, False), norm(x), rtol=1e-5, atol=1e-5)
