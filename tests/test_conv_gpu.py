"""NHWC convolution / pooling / batch-norm kernels against torch.nn.functional in fp32."""
import pytest
import torch
import torch.nn.functional as F

from scirust_b200.ops import _lib, conv as C

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _close(a, b, tol=3e-2):
    err = (a.float() - b.float()).abs().max().item()
    lim = tol * max(1.0, b.float().abs().max().item())
    assert err <= lim, f"{err} > {lim}"


@pytest.mark.parametrize("B,Cin,H,W,Cout,k,stride,pad", [(2, 1, 28, 28, 32, 3, 1, 0), (3, 32, 26, 26, 64, 3, 1, 0),
                                                         (2, 64, 16, 16, 128, 3, 2, 1), (2, 3, 32, 32, 64, 3, 1, 1),
                                                         (2, 64, 8, 8, 128, 1, 2, 0)])
def test_conv_forward_backward(B, Cin, H, W, Cout, k, stride, pad):
    g = torch.Generator(device="cuda").manual_seed(0)
    x4 = torch.randn(B, Cin, H, W, generator=g, device="cuda").to(BF)
    w_ref = (torch.randn(Cout, Cin * k * k, generator=g, device="cuda") * 0.1).to(BF)
    rows, geom = C.nchw_to_rows(x4)
    rows.requires_grad_(True)
    wp = C.pack_conv_weight(w_ref, Cin, k).requires_grad_(True)
    y, og = C.conv2d(rows, wp, geom, k, stride, pad)
    _lib.check_status()
    xr = x4.float().requires_grad_(True)
    wr = w_ref.float().reshape(Cout, Cin, k, k).requires_grad_(True)
    yr = F.conv2d(xr, wr, stride=stride, padding=pad)
    _close(C.rows_to_nchw(y, og), yr)
    dy4 = torch.randn(yr.shape, generator=g, device="cuda").to(BF)
    y.backward(C.nchw_to_rows(dy4)[0])
    yr.backward(dy4.float())
    _close(C.rows_to_nchw(rows.grad, geom), xr.grad)
    _close(C.unpack_conv_weight(wp.grad, Cin, k), wr.grad.reshape(Cout, -1))


def test_maxpool_and_batchnorm():
    g = torch.Generator(device="cuda").manual_seed(1)
    x4 = torch.randn(4, 16, 12, 12, generator=g, device="cuda").to(BF)
    rows, geom = C.nchw_to_rows(x4)
    rows.requires_grad_(True)
    y, og = C.maxpool2d(rows, geom, 2, 2)
    xr = x4.float().requires_grad_(True)
    yr = F.max_pool2d(xr, 2, 2)
    assert torch.equal(C.rows_to_nchw(y, og).float(), yr.to(BF).float())
    dy = torch.randn(yr.shape, generator=g, device="cuda").to(BF)
    y.backward(C.nchw_to_rows(dy)[0])
    yr.backward(dy.float())
    _close(C.rows_to_nchw(rows.grad, geom), xr.grad, 1e-2)
    # overlapping windows
    y2, og2 = C.maxpool2d(rows.detach(), geom, 3, 2)
    assert torch.equal(C.rows_to_nchw(y2, og2).float(), F.max_pool2d(x4.float(), 3, 2).to(BF).float())

    for relu in (False, True):
        xb = rows.detach().clone().requires_grad_(True)
        gamma = (torch.rand(16, device="cuda") + 0.5).requires_grad_(True)
        beta = torch.randn(16, device="cuda").requires_grad_(True)
        rm, rv = torch.zeros(16, device="cuda"), torch.ones(16, device="cuda")
        yb = C.batchnorm(xb, gamma, beta, rm, rv, relu=relu, training=True)
        x2 = rows.detach().float().clone().requires_grad_(True)
        g2, b2 = gamma.detach().clone().requires_grad_(True), beta.detach().clone().requires_grad_(True)
        rm2, rv2 = torch.zeros(16, device="cuda"), torch.ones(16, device="cuda")
        y2 = F.batch_norm(x2.t().unsqueeze(0), rm2, rv2, g2, b2, True, 0.1, 1e-5)[0].t()
        if relu:
            y2 = torch.relu(y2)
        _close(yb, y2)
        assert torch.allclose(rm, rm2, atol=2e-3) and torch.allclose(rv, rv2, atol=5e-3)
        d = torch.randn(y2.shape, generator=g, device="cuda").to(BF)
        yb.backward(d)
        y2.backward(d.float())
        _close(xb.grad, x2.grad, 5e-2)
        assert torch.allclose(gamma.grad, g2.grad, rtol=3e-2, atol=0.3)
        assert torch.allclose(beta.grad, b2.grad, rtol=3e-2, atol=0.3)
        ye = C.batchnorm(rows.detach(), gamma.detach(), beta.detach(), rm, rv, relu=relu, training=False)
        yr2 = F.batch_norm(rows.detach().float().t().unsqueeze(0), rm, rv, gamma.detach(), beta.detach(), False)[0].t()
        _close(ye, torch.relu(yr2) if relu else yr2)


def test_cnn_models_train_on_gpu():
    from scirust_b200.models.cnn import MnistCNN, ResNet18
    from scirust_b200.parallel.ddp import FlatDataParallel
    torch.manual_seed(0)
    for model, x in ((MnistCNN().cuda(), torch.rand(32, 784, device="cuda")),
                     (ResNet18().cuda(), torch.randn(16, 3 * 32 * 32, device="cuda"))):
        y = torch.randint(0, 10, (x.shape[0],), device="cuda")
        dp = FlatDataParallel(model, optimizer="sgd", lr=0.01, momentum=0.9)
        losses = []
        for _ in range(8):
            loss = F.cross_entropy(dp(x), y)
            loss.backward()
            dp.step()
            losses.append(float(loss.detach()))
        _lib.check_status()
        assert losses[-1] < losses[0], losses
