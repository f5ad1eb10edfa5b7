"""Convolutional ops on NHWC bf16 activations (csrc/conv.cu + the tcgen05 GEMM): explicit-GEMM
convolution (im2col -> GEMM, col2im for the input gradient, transposed GEMM for the weight
gradient), max pooling, BatchNorm2d with optional fused ReLU. Activations are ``[B*H*W, C]``
matrices; ``ConvGeom`` carries the spatial shape. CPU tensors run the fp32 PyTorch statement
(``torch.nn.functional``), which is also the oracle of the GPU tests."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib
from . import gemm as G

BF = torch.bfloat16
vp, i32, f32, sz = _lib.vp, _lib.i32, _lib.f32, _lib.sz
_lib.register("sb_im2col_nhwc", [vp, vp] + [i32] * 11 + [vp])
_lib.register("sb_col2im_nhwc", [vp, vp] + [i32] * 11 + [vp])
_lib.register("sb_maxpool_fwd", [vp, vp, vp] + [i32] * 8 + [vp])
_lib.register("sb_maxpool_bwd", [vp, vp, vp] + [i32] * 8 + [vp])
_lib.register("sb_colstats", [vp, vp, vp, vp, vp, i32, i32, vp])
_lib.register("sb_bn_fwd", [vp] * 10 + [i32, i32, f32, f32, i32, i32, vp])
_lib.register("sb_bn_bwd", [vp] * 10 + [i32, i32, vp])
_lib.register("sb_relu_mask", [vp, vp, vp, sz, vp])
_lib.register("sb_bias_act", [vp, vp, vp, sz, i32, i32, vp])


@dataclass(frozen=True)
class ConvGeom:
    B: int
    H: int
    W: int
    C: int

    @property
    def rows(self):
        return self.B * self.H * self.W


def _pad8(n):
    return (n + 7) // 8 * 8


def nchw_to_rows(x4: torch.Tensor):
    B, C, H, W = x4.shape
    return x4.permute(0, 2, 3, 1).reshape(B * H * W, C).contiguous(), ConvGeom(B, H, W, C)


def rows_to_nchw(x: torch.Tensor, g: ConvGeom):
    return x.reshape(g.B, g.H, g.W, g.C).permute(0, 3, 1, 2).contiguous()


def pack_conv_weight(w_ref: torch.Tensor, in_c: int, k: int) -> torch.Tensor:
    """Reference layout ``(out_c, in_c*k*k)`` with (c, kh, kw) order -> ``[out_c, pad8(k*k*in_c)]`` with
    (kh, kw, c) order, the column order of the NHWC patches."""
    oc = w_ref.shape[0]
    w = w_ref.reshape(oc, in_c, k, k).permute(0, 2, 3, 1).reshape(oc, k * k * in_c)
    out = torch.zeros((oc, _pad8(k * k * in_c)), dtype=w_ref.dtype, device=w_ref.device)
    out[:, : k * k * in_c] = w
    return out


def unpack_conv_weight(wp: torch.Tensor, in_c: int, k: int) -> torch.Tensor:
    oc = wp.shape[0]
    return wp[:, : k * k * in_c].reshape(oc, k, k, in_c).permute(0, 3, 1, 2).reshape(oc, in_c * k * k)


class _Conv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wp, geom, k, stride, pad):
        B, H, W, C = geom.B, geom.H, geom.W, geom.C
        OH, OW = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
        Kp = wp.shape[1]
        col = _lib.empty((B * OH * OW, Kp), BF, x.device)
        _lib.call("sb_im2col_nhwc", x.data_ptr(), col.data_ptr(), B, H, W, C, k, k, stride, pad, OH, OW, Kp,
                  _lib.stream())
        G.launch_count += 1
        y = G.matmul_nt(col, wp)
        ctx.save_for_backward(col, wp)
        ctx.meta = (geom, k, stride, pad, OH, OW)
        return y

    @staticmethod
    def backward(ctx, dy):
        col, wp = ctx.saved_tensors
        geom, k, stride, pad, OH, OW = ctx.meta
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[1]:
            dw = G.matmul_tn(dy, col)                         # [oc, Kp] = dy^T col
        if ctx.needs_input_grad[0]:
            dcol = G.matmul_nn(dy, wp)                        # [M, Kp]
            dx = _lib.empty((geom.rows, geom.C), BF, dy.device)
            _lib.call("sb_col2im_nhwc", dcol.data_ptr(), dx.data_ptr(), geom.B, geom.H, geom.W, geom.C, k, k, stride,
                      pad, OH, OW, wp.shape[1], _lib.stream())
            G.launch_count += 1
        return dx, dw, None, None, None, None


def conv2d(x, wp, geom: ConvGeom, k: int, stride: int = 1, pad: int = 0):
    """x [B*H*W, C], wp packed weight [oc, pad8(k*k*C)] -> (y [B*OH*OW, oc], geometry of y)."""
    OH, OW = (geom.H + 2 * pad - k) // stride + 1, (geom.W + 2 * pad - k) // stride + 1
    og = ConvGeom(geom.B, OH, OW, wp.shape[0])
    if not x.is_cuda:
        w4 = wp[:, : k * k * geom.C].reshape(wp.shape[0], k, k, geom.C).permute(0, 3, 1, 2)
        y4 = F.conv2d(rows_to_nchw(x.float(), geom), w4.float(), stride=stride, padding=pad)
        return nchw_to_rows(y4.to(x.dtype))[0], og
    return _Conv.apply(x.contiguous(), wp, geom, k, stride, pad), og


class _MaxPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, geom, k, stride):
        B, H, W, C = geom.B, geom.H, geom.W, geom.C
        OH, OW = (H - k) // stride + 1, (W - k) // stride + 1
        y = _lib.empty((B * OH * OW, C), BF, x.device)
        arg = _lib.empty((B * OH * OW, C), torch.uint8, x.device)
        _lib.call("sb_maxpool_fwd", x.data_ptr(), y.data_ptr(), arg.data_ptr(), B, H, W, C, k, stride, OH, OW,
                  _lib.stream())
        G.launch_count += 1
        ctx.save_for_backward(arg)
        ctx.meta = (geom, k, stride, OH, OW)
        return y

    @staticmethod
    def backward(ctx, dy):
        (arg,) = ctx.saved_tensors
        geom, k, stride, OH, OW = ctx.meta
        dx = _lib.empty((geom.rows, geom.C), BF, dy.device)
        _lib.call("sb_maxpool_bwd", dy.contiguous().data_ptr(), arg.data_ptr(), dx.data_ptr(), geom.B, geom.H, geom.W,
                  geom.C, k, stride, OH, OW, _lib.stream())
        G.launch_count += 1
        return dx, None, None, None


def maxpool2d(x, geom: ConvGeom, k: int, stride: int):
    OH, OW = (geom.H - k) // stride + 1, (geom.W - k) // stride + 1
    og = ConvGeom(geom.B, OH, OW, geom.C)
    if not x.is_cuda:
        return nchw_to_rows(F.max_pool2d(rows_to_nchw(x, geom), k, stride))[0], og
    return _MaxPool.apply(x.contiguous(), geom, k, stride), og


def _colstats(a, b):
    rows, C = a.shape
    part = torch.empty(2 * ((rows + 255) // 256) * C, dtype=torch.float32, device=a.device)
    s1 = _lib.empty(C, torch.float32, a.device)
    s2 = _lib.empty(C, torch.float32, a.device)
    _lib.call("sb_colstats", a.data_ptr(), b.data_ptr(), part.data_ptr(), s1.data_ptr(), s2.data_ptr(), rows, C,
              _lib.stream())
    G.launch_count += 2
    return s1, s2


class _BatchNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, run_mean, run_var, eps, momentum, relu, training):
        rows, C = x.shape
        mean = _lib.empty(C, torch.float32, x.device)
        inv = _lib.empty(C, torch.float32, x.device)
        if training:
            s1, s2 = _colstats(x, x)
        else:
            s1 = s2 = None
            mean.copy_(run_mean)
            inv.copy_(torch.rsqrt(run_var + eps))
        y = torch.empty_like(x)
        _lib.call("sb_bn_fwd", x.data_ptr(), _lib.ptr(s1), _lib.ptr(s2), gamma.data_ptr(), beta.data_ptr(),
                  mean.data_ptr(), inv.data_ptr(), _lib.ptr(run_mean) if training else None,
                  _lib.ptr(run_var) if training else None, y.data_ptr(), rows, C, float(eps), float(momentum),
                  int(relu), int(training), _lib.stream())
        G.launch_count += 2
        ctx.save_for_backward(x, y, gamma, mean, inv)
        ctx.relu = relu
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, gamma, mean, inv = ctx.saved_tensors
        rows, C = x.shape
        dy = dy.contiguous()
        g = dy
        if ctx.relu:
            g = torch.empty_like(dy)
            _lib.call("sb_relu_mask", dy.data_ptr(), y.data_ptr(), g.data_ptr(), dy.numel(), _lib.stream())
        sg, sgx = _colstats(g, x)
        dgamma = _lib.empty(C, torch.float32, x.device)
        dbeta = _lib.empty(C, torch.float32, x.device)
        dx = torch.empty_like(x)
        _lib.call("sb_bn_bwd", g.data_ptr(), x.data_ptr(), sg.data_ptr(), sgx.data_ptr(), mean.data_ptr(),
                  inv.data_ptr(), gamma.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), dx.data_ptr(), rows, C,
                  _lib.stream())
        G.launch_count += 3
        return dx, dgamma, dbeta, None, None, None, None, None, None


def batchnorm(x, gamma, beta, run_mean, run_var, eps=1e-5, momentum=0.1, relu=False, training=True):
    """Per-channel batch norm of [rows, C] (fp32 gamma/beta/running stats), optional fused ReLU."""
    if not x.is_cuda:
        y = F.batch_norm(x.float().t().unsqueeze(0), run_mean, run_var, gamma, beta, training, momentum, eps)[0].t()
        return (torch.relu(y) if relu else y).to(x.dtype)
    return _BatchNorm.apply(x.contiguous(), gamma, beta, run_mean, run_var, eps, momentum, relu, training)


def bias_act(x, bias, relu=False):
    """y = act(x + bias[c]) with fp32 bias; differentiable through PyTorch for the bias."""
    if not x.is_cuda or torch.is_grad_enabled():
        y = x + bias.to(x.dtype) if bias is not None else x
        return torch.relu(y) if relu else y
    y = torch.empty_like(x)
    _lib.call("sb_bias_act", x.data_ptr(), _lib.ptr(bias), y.data_ptr(), x.numel(), x.shape[1], int(relu), _lib.stream())
    return y
