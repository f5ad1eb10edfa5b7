"""Neural-network layers with SciRust's names, shapes and state-dict keys, on ``torch.nn.Module``.

Conventions taken from the reference (scirust-core/src/nn):

* ``Linear``: ``y = x.W + b`` with ``W (in, out)``, ``b (1, out)``; keys ``weight``, ``bias``
  (nn/linear.rs:24-139).
* ``Conv2d`` / ``MaxPool2d``: images travel flattened as ``(B, C*H*W)`` in NCHW order; conv weight is
  ``(out_c, in_c*K*K)``; ``Padding.SAME`` / ``VALID`` (nn/conv2d.rs:13-208, nn/conv_utils.rs:19-120,
  nn/pool.rs).
* ``LayerNorm`` keys ``{name}/gamma``, ``{name}/beta`` (nn/layer_norm.rs:92-110); ``RMSNorm`` key
  ``{name}/weight`` (scirust-sciagent/src/norm.rs:45-75); ``BatchNorm1d/2d`` with running statistics,
  momentum 0.1, eps 1e-5, unbiased running variance (nn/batch_norm_2d.rs:18-90,177-190).
* ``Embedding`` key ``{name}.weight`` (nn/embedding.rs:14-110).
* ``Sequential`` prefixes child keys with the layer index ``"{i}.{k}"`` (nn/sequential.rs:105-116).
* ``Module`` surface: ``forward``, ``train``, ``parameters``, ``state_dict_ref`` /
  ``load_state_dict_ref`` (2-D fp32 tensors under the reference's names; nn/module.rs:31-84).

Layers accept a ``torch.Tensor`` or a tape ``Var`` (the result is then a ``Var`` on the same tape).
On CUDA bf16 inputs ``Linear`` and ``RMSNorm`` run the native kernels of ``scirust_b200.ops``.
"""
from __future__ import annotations

import enum
import math

import torch
import torch.nn as tnn
import torch.nn.functional as F

from .. import ops
from ..autodiff.tape import Var
from . import init as I
from .rng import PcgEngine


class Padding(enum.Enum):
    VALID = 0
    SAME = 1


def _unwrap(x):
    return (x.t, x) if isinstance(x, Var) else (x, None)


def _wrap(y, var):
    return var._new(y) if var is not None else y


class Module(tnn.Module):
    """Base class: adds reference-style state dicts on top of ``torch.nn.Module``."""

    ref_name = ""

    def with_name(self, name: str):
        self.ref_name = name
        return self

    def state_dict_ref(self) -> dict:
        return {}

    def load_state_dict_ref(self, sd: dict) -> None:
        pass

    def parameter_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def __call__(self, x, *a, **kw):
        t, var = _unwrap(x)
        return _wrap(super().__call__(t, *a, **kw), var)


class _LinearFn(torch.autograd.Function):
    """bf16 CUDA path: forward / input-gradient / weight-gradient on the tcgen05 GEMM."""

    @staticmethod
    def forward(ctx, x, w, b):
        ctx.save_for_backward(x, w)
        ctx.has_bias = b is not None
        # the bias is added in the GEMM epilogue (the residual operand with a zero row pitch)
        return ops.matmul_nn(x, w, bias=b.reshape(-1).contiguous() if b is not None else None)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = ops.matmul_nt(dy, w) if ctx.needs_input_grad[0] else None
        dw = ops.matmul_tn(x, dy) if ctx.needs_input_grad[1] else None
        db = dy.float().sum(0, keepdim=True).to(dy.dtype) if ctx.has_bias else None
        return dx, dw, db


class Linear(Module):
    def __init__(self, in_features: int, out_features: int, weight_init: I.Initializer | None = None,
                 bias_init: I.Initializer | None = None, rng: PcgEngine | None = None, bias: bool = True):
        super().__init__()
        rng = rng or PcgEngine(0)
        wi = weight_init or I.KaimingNormal()
        self.in_features, self.out_features = in_features, out_features
        self.weight = tnn.Parameter(wi.fill((in_features, out_features), in_features, out_features, rng))
        if bias:
            bi = bias_init or I.Zeros()
            self.bias = tnn.Parameter(bi.fill((1, out_features), in_features, out_features, rng))
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        if x.shape[-1] != self.in_features:
            raise ValueError(f"Linear: expected {self.in_features} input features, got {x.shape[-1]}")
        if x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and self.out_features % 8 == 0 \
                and self.in_features % 8 == 0:
            return _LinearFn.apply(x.contiguous(), self.weight, self.bias)
        y = x @ self.weight
        return y + self.bias if self.bias is not None else y

    def state_dict_ref(self):
        p = f"{self.ref_name}." if self.ref_name else ""
        sd = {f"{p}weight": self.weight.detach().float().cpu()}
        if self.bias is not None:
            sd[f"{p}bias"] = self.bias.detach().float().cpu()
        return sd

    def load_state_dict_ref(self, sd):
        p = f"{self.ref_name}." if self.ref_name else ""
        w = torch.as_tensor(sd[f"{p}weight"])
        if tuple(w.shape) != tuple(self.weight.shape):
            raise ValueError(f"Linear: weight shape {tuple(w.shape)} != {tuple(self.weight.shape)}")
        with torch.no_grad():
            self.weight.copy_(w)
            if self.bias is not None and f"{p}bias" in sd:
                self.bias.copy_(torch.as_tensor(sd[f"{p}bias"]).reshape(1, -1))


class ReLU(Module):
    def forward(self, x): return torch.relu(x)


class Sigmoid(Module):
    def forward(self, x): return torch.sigmoid(x)


class Tanh(Module):
    def forward(self, x): return torch.tanh(x)


class GELU(Module):
    def forward(self, x): return F.gelu(x)


class SiLU(Module):
    def forward(self, x): return F.silu(x)


class Dropout(Module):
    def __init__(self, p: float = 0.5, seed: int = 0):
        super().__init__()
        self.p = p
        self._gen = torch.Generator().manual_seed(seed)

    def forward(self, x):
        if not self.training or self.p <= 0:
            return x
        keep = (torch.rand(x.shape, generator=self._gen) >= self.p).to(x.device, x.dtype)
        return x * keep / (1.0 - self.p)


class Embedding(Module):
    def __init__(self, vocab: int, dim: int, rng: PcgEngine | None = None, std: float = 0.02):
        super().__init__()
        rng = rng or PcgEngine(0)
        self.weight = tnn.Parameter(rng.fill_normal((vocab, dim), 0.0, std))

    def forward(self, idx):
        idx = torch.as_tensor(idx, dtype=torch.long, device=self.weight.device)
        if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= self.weight.shape[0]):
            raise IndexError("Embedding: token id out of range")
        return self.weight[idx.reshape(-1)]

    def state_dict_ref(self):
        return {f"{self.ref_name}.weight" if self.ref_name else "weight": self.weight.detach().float().cpu()}

    def load_state_dict_ref(self, sd):
        with torch.no_grad():
            self.weight.copy_(torch.as_tensor(sd[f"{self.ref_name}.weight" if self.ref_name else "weight"]))


class LayerNorm(Module):
    def __init__(self, d_model: int, eps: float = 1e-5):
        super().__init__()
        self.d_model, self.eps = d_model, eps
        self.gamma = tnn.Parameter(torch.ones(1, d_model))
        self.beta = tnn.Parameter(torch.zeros(1, d_model))

    def forward(self, x):
        return F.layer_norm(x, (self.d_model,), self.gamma.reshape(-1), self.beta.reshape(-1), self.eps)

    def state_dict_ref(self):
        n = self.ref_name or "layer_norm"
        return {f"{n}/gamma": self.gamma.detach().float().cpu(), f"{n}/beta": self.beta.detach().float().cpu()}

    def load_state_dict_ref(self, sd):
        n = self.ref_name or "layer_norm"
        with torch.no_grad():
            self.gamma.copy_(torch.as_tensor(sd[f"{n}/gamma"]).reshape(1, -1))
            self.beta.copy_(torch.as_tensor(sd[f"{n}/beta"]).reshape(1, -1))


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        y, inv = ops.rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, inv)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, inv = ctx.saved_tensors
        dx, dw = ops.rmsnorm_bwd(dy.contiguous(), x, w, inv)
        return dx, dw.to(w.dtype), None


class RMSNorm(Module):
    def __init__(self, d_model: int, eps: float = 1e-5):
        super().__init__()
        self.d_model, self.eps = d_model, eps
        self.weight = tnn.Parameter(torch.ones(1, d_model))

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and self.d_model % 8 == 0:
            return _RMSNormFn.apply(x.contiguous(), self.weight.reshape(-1).to(torch.bfloat16), self.eps)
        inv = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)
        return x * inv * self.weight.reshape(-1)

    def state_dict_ref(self):
        return {f"{self.ref_name or 'rms_norm'}/weight": self.weight.detach().float().cpu()}

    def load_state_dict_ref(self, sd):
        with torch.no_grad():
            self.weight.copy_(torch.as_tensor(sd[f"{self.ref_name or 'rms_norm'}/weight"]).reshape(1, -1))


class _BatchNorm(Module):
    def __init__(self, channels: int, eps: float = 1e-5, momentum: float = 0.1):
        super().__init__()
        self.channels, self.eps, self.momentum = channels, eps, momentum
        self.gamma = tnn.Parameter(torch.ones(1, channels))
        self.beta = tnn.Parameter(torch.zeros(1, channels))
        self.register_buffer("running_mean", torch.zeros(1, channels))
        self.register_buffer("running_var", torch.ones(1, channels))

    def _norm(self, x4):
        # x4: (B, C, H, W); torch's functional batch norm keeps running variance unbiased (Bessel)
        return F.batch_norm(x4, self.running_mean.reshape(-1), self.running_var.reshape(-1), self.gamma.reshape(-1),
                            self.beta.reshape(-1), self.training, self.momentum, self.eps)

    def state_dict_ref(self):
        n = self.ref_name or "batch_norm"
        return {f"{n}/gamma": self.gamma.detach().float().cpu(), f"{n}/beta": self.beta.detach().float().cpu(),
                f"{n}/running_mean": self.running_mean.float().cpu(), f"{n}/running_var": self.running_var.float().cpu()}

    def load_state_dict_ref(self, sd):
        n = self.ref_name or "batch_norm"
        with torch.no_grad():
            self.gamma.copy_(torch.as_tensor(sd[f"{n}/gamma"]).reshape(1, -1))
            self.beta.copy_(torch.as_tensor(sd[f"{n}/beta"]).reshape(1, -1))
            if f"{n}/running_mean" in sd:
                self.running_mean.copy_(torch.as_tensor(sd[f"{n}/running_mean"]).reshape(1, -1))
                self.running_var.copy_(torch.as_tensor(sd[f"{n}/running_var"]).reshape(1, -1))


class BatchNorm1d(_BatchNorm):
    def forward(self, x):
        return self._norm(x.reshape(x.shape[0], self.channels, 1, 1)).reshape(x.shape)


class BatchNorm2d(_BatchNorm):
    """Input ``(B, C*H*W)``; ``h, w`` are inferred from the width when not given."""

    def __init__(self, channels: int, h: int | None = None, w: int | None = None, **kw):
        super().__init__(channels, **kw)
        self.h, self.w = h, w

    def forward(self, x):
        B = x.shape[0]
        hw = x.shape[1] // self.channels
        h = self.h or int(round(math.sqrt(hw)))
        w = self.w or hw // h
        return self._norm(x.reshape(B, self.channels, h, w)).reshape(B, -1)


class Conv2d(Module):
    def __init__(self, in_c: int, out_c: int, kernel: int, stride: int = 1, padding: Padding = Padding.VALID,
                 in_h: int = 0, in_w: int = 0, rng: PcgEngine | None = None, bias: bool = True):
        super().__init__()
        rng = rng or PcgEngine(0)
        self.in_c, self.out_c, self.kernel, self.stride, self.padding = in_c, out_c, kernel, stride, padding
        self.in_h, self.in_w = in_h, in_w
        fan_in = in_c * kernel * kernel
        self.weight = tnn.Parameter(I.KaimingNormal().fill((out_c, fan_in), fan_in, out_c, rng))
        self.bias = tnn.Parameter(torch.zeros(1, out_c)) if bias else None

    def out_hw(self, h=None, w=None):
        h, w = h or self.in_h, w or self.in_w
        if self.padding == Padding.SAME:
            return (h + self.stride - 1) // self.stride, (w + self.stride - 1) // self.stride
        return (h - self.kernel) // self.stride + 1, (w - self.kernel) // self.stride + 1

    def forward(self, x, h: int | None = None, w: int | None = None):
        h, w = h or self.in_h, w or self.in_w
        B = x.shape[0]
        if x.shape[1] != self.in_c * h * w:
            raise ValueError(f"Conv2d: input width {x.shape[1]} != {self.in_c}*{h}*{w}")
        x4 = x.reshape(B, self.in_c, h, w)
        k = self.kernel
        if self.padding == Padding.SAME:
            oh, ow = self.out_hw(h, w)
            ph = max((oh - 1) * self.stride + k - h, 0)
            pw = max((ow - 1) * self.stride + k - w, 0)
            x4 = F.pad(x4, (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2))
        y = F.conv2d(x4, self.weight.reshape(self.out_c, self.in_c, k, k).to(x4.dtype),
                     self.bias.reshape(-1).to(x4.dtype) if self.bias is not None else None, stride=self.stride)
        return y.reshape(B, -1)

    def state_dict_ref(self):
        p = f"{self.ref_name}." if self.ref_name else ""
        sd = {f"{p}weight": self.weight.detach().float().cpu()}
        if self.bias is not None:
            sd[f"{p}bias"] = self.bias.detach().float().cpu()
        return sd

    def load_state_dict_ref(self, sd):
        p = f"{self.ref_name}." if self.ref_name else ""
        with torch.no_grad():
            self.weight.copy_(torch.as_tensor(sd[f"{p}weight"]))
            if self.bias is not None and f"{p}bias" in sd:
                self.bias.copy_(torch.as_tensor(sd[f"{p}bias"]).reshape(1, -1))


class ConvTranspose2d(Module):
    def __init__(self, in_c, out_c, kernel, stride=1, in_h=0, in_w=0, rng=None):
        super().__init__()
        rng = rng or PcgEngine(0)
        self.in_c, self.out_c, self.kernel, self.stride, self.in_h, self.in_w = in_c, out_c, kernel, stride, in_h, in_w
        fan_in = in_c * kernel * kernel
        self.weight = tnn.Parameter(I.KaimingNormal().fill((in_c, out_c * kernel * kernel), fan_in, out_c, rng))
        self.bias = tnn.Parameter(torch.zeros(1, out_c))

    def forward(self, x, h=None, w=None):
        h, w = h or self.in_h, w or self.in_w
        B = x.shape[0]
        y = F.conv_transpose2d(x.reshape(B, self.in_c, h, w),
                               self.weight.reshape(self.in_c, self.out_c, self.kernel, self.kernel),
                               self.bias.reshape(-1), stride=self.stride)
        return y.reshape(B, -1)


class MaxPool2d(Module):
    def __init__(self, kernel: int, stride: int, c: int, h: int, w: int):
        super().__init__()
        self.kernel, self.stride, self.c, self.h, self.w = kernel, stride, c, h, w

    def out_hw(self):
        return (self.h - self.kernel) // self.stride + 1, (self.w - self.kernel) // self.stride + 1

    def forward(self, x):
        B = x.shape[0]
        return F.max_pool2d(x.reshape(B, self.c, self.h, self.w), self.kernel, self.stride).reshape(B, -1)


class GlobalAvgPool2d(Module):
    def __init__(self, c: int):
        super().__init__()
        self.c = c

    def forward(self, x):
        B = x.shape[0]
        return x.reshape(B, self.c, -1).mean(-1)


class Sequential(Module):
    def __init__(self, *layers):
        super().__init__()
        self.layers = tnn.ModuleList(layers)

    def add(self, layer):
        self.layers.append(layer)
        return self

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x

    def state_dict_ref(self):
        sd = {}
        for i, l in enumerate(self.layers):
            if isinstance(l, Module):
                for k, v in l.state_dict_ref().items():
                    sd[f"{i}.{k}"] = v
        return sd

    def load_state_dict_ref(self, sd):
        for i, l in enumerate(self.layers):
            if isinstance(l, Module):
                pre = f"{i}."
                sub = {k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}
                if sub or l.state_dict_ref():
                    l.load_state_dict_ref(sub)


class SinusoidalPositionalEncoding(Module):
    def __init__(self, d_model: int, max_len: int = 4096):
        super().__init__()
        pos = torch.arange(max_len)[:, None].float()
        div = torch.exp(torch.arange(0, d_model, 2).float() * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)[:, : d_model // 2]
        self.register_buffer("pe", pe)

    def forward(self, x, seq_len: int | None = None):
        n = x.shape[0] if seq_len is None else seq_len
        reps = x.shape[0] // n
        return x + self.pe[:n].repeat(reps, 1).to(x.dtype)


def rope_frequencies(head_dim: int, theta: float = 10000.0) -> torch.Tensor:
    p = torch.arange(head_dim // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * p / head_dim).float()


def yarn_frequencies(head_dim: int, theta: float, scale: float, orig_len: int, beta_fast: float = 32.0,
                     beta_slow: float = 1.0):
    """YaRN NTK-by-parts: high-frequency pairs keep their rotation, low-frequency pairs are
    interpolated by 1/scale, with a linear ramp between the two wavelength thresholds; also returns
    the attention temperature 0.1 ln(scale) + 1 (scirust-core/src/nn/yarn.rs:1-241)."""
    inv = rope_frequencies(head_dim, theta).double()

    def corr_dim(n_rot):
        return head_dim * math.log(orig_len / (n_rot * 2 * math.pi)) / (2 * math.log(theta))
    lo = max(math.floor(corr_dim(beta_fast)), 0)
    hi = min(math.ceil(corr_dim(beta_slow)), head_dim // 2 - 1)
    idx = torch.arange(head_dim // 2, dtype=torch.float64)
    ramp = ((idx - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
    blended = inv / scale * ramp + inv * (1 - ramp)
    mscale = 0.1 * math.log(scale) + 1.0 if scale > 1 else 1.0
    return blended.float(), mscale
