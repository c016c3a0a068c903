"""Host-side mirror of the reference's Module interface for the hot-path layers.

Same names, argument order and behaviour as the C vtable (src/nn.h:159-174):
    forward(in, out, batch, ctx)
    backward(in, out, grad_out, grad_in, batch, ctx)   -- `out` may be None, parameter
                                                          gradients are overwritten
    parameters(pl)                                     -- appends (param, grad, size)
    free()
and the constructors of src/nn.h:185-198, 273-283.  TEST SCAFFOLDING: the production host side is the
reference's own C modules linked against the library (and csrc/host/*.c); this mirror exists so that
tests/test_modules_gpu.py can drive the same call sequences from Python.
All compute goes through the C ABI; dense products (mp_linear) go to cuBLAS via torch.matmul
exactly as the reference sends them to cublasSgemm.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

import importlib

ops = importlib.import_module("cuda-c-diffusion_b200.ops")


@dataclass
class Context:
    """src/nn.h:71-77 without the library handles: the stream is torch's current stream."""
    cond: list = field(default_factory=list)


@dataclass
class Param:
    param: torch.Tensor
    grad: torch.Tensor
    size: int


class ParamList(list):
    """src/nn.h:145-153"""

    def add(self, param, grad, size):
        self.append(Param(param, grad, size))


class Module:
    name = "module"
    in_dim = out_dim = 0

    def forward(self, inp, out, batch, ctx=None):
        raise NotImplementedError

    def backward(self, inp, out, grad_out, grad_in, batch, ctx=None):
        raise NotImplementedError

    def parameters(self, pl):
        pass

    def free(self):
        pass


class Activation(Module):
    """activation_create(dim, act) -- src/activation.c"""
    name = "activation"

    def __init__(self, dim, act):
        self.in_dim = self.out_dim = dim
        self.act = act

    def forward(self, inp, out, batch, ctx=None):
        ops.activation_forward(inp, self.act, out=out)

    def backward(self, inp, out, grad_out, grad_in, batch, ctx=None):
        ops.activation_backward(grad_out, inp, self.act, grad_in=grad_in)


class _AffineNorm(Module):
    def _alloc_affine(self, C, device):
        self.gamma = torch.ones(C, device=device)
        self.beta = torch.zeros(C, device=device)
        self.ggamma = torch.zeros(C, device=device)
        self.gbeta = torch.zeros(C, device=device)

    def parameters(self, pl):
        pl.add(self.gamma, self.ggamma, self.gamma.numel())
        pl.add(self.beta, self.gbeta, self.beta.numel())


class SpatialGroupNorm(_AffineNorm):
    """spatial_groupnorm_create(C, num_groups, H, W, max_batch) -- src/groupnorm.c; eps = 1e-5.
    `act` (not in the reference) selects the fused GroupNorm+activation entry points."""
    name = "groupnorm"

    def __init__(self, C, num_groups, H, W, max_batch, device="cuda", act=None):
        if C % num_groups:
            raise ValueError("groupnorm: C must be divisible by num_groups")
        self.C, self.G, self.H, self.W, self.max_batch, self.eps, self.act = C, num_groups, H, W, max_batch, 1e-5, act
        self.in_dim = self.out_dim = H * W * C
        self._alloc_affine(C, device)
        self.mu = torch.empty(max_batch * num_groups, device=device)
        self.rstd = torch.empty_like(self.mu)

    def forward(self, inp, out, batch, ctx=None):
        lib, P, st = ops._lib(), ops._p, ops._stream()
        if self.act is None:
            lib.launch_groupnorm_forward(P(out), P(self.mu), P(self.rstd), P(inp), P(self.gamma), P(self.beta), batch,
                                         self.H * self.W, self.C, self.G, self.eps, st)
        else:
            lib.launch_groupnorm_act_forward(P(out), P(self.mu), P(self.rstd), P(inp), P(self.gamma), P(self.beta),
                                             batch, self.H * self.W, self.C, self.G, self.eps, ops._act(self.act), st)

    def backward(self, inp, out, grad_out, grad_in, batch, ctx=None):
        lib, P, st = ops._lib(), ops._p, ops._stream()
        if self.act is None:
            lib.launch_groupnorm_backward(P(grad_in), P(self.ggamma), P(self.gbeta), P(grad_out), P(inp), P(self.gamma),
                                          P(self.mu), P(self.rstd), batch, self.H * self.W, self.C, self.G, st)
        else:
            lib.launch_groupnorm_act_backward(P(grad_in), P(self.ggamma), P(self.gbeta), P(grad_out), P(inp),
                                              P(self.gamma), P(self.beta), P(self.mu), P(self.rstd), batch,
                                              self.H * self.W, self.C, self.G, ops._act(self.act), st)


class LayerNorm(_AffineNorm):
    """layernorm_create(dim, max_batch) -- src/layernorm.c; eps = 1e-5"""
    name = "layernorm"

    def __init__(self, dim, max_batch, device="cuda"):
        self.C, self.max_batch, self.eps = dim, max_batch, 1e-5
        self.in_dim = self.out_dim = dim
        self._alloc_affine(dim, device)
        self.mu = torch.empty(max_batch, device=device)
        self.rstd = torch.empty_like(self.mu)

    def forward(self, inp, out, batch, ctx=None):
        P = ops._p
        ops._lib().launch_layernorm_forward(P(out), P(self.mu), P(self.rstd), P(inp), P(self.gamma), P(self.beta),
                                            batch, self.C, self.eps, ops._stream())

    def backward(self, inp, out, grad_out, grad_in, batch, ctx=None):
        P = ops._p
        ops._lib().launch_layernorm_backward(P(grad_in), P(self.ggamma), P(self.gbeta), P(grad_out), P(inp),
                                             P(self.gamma), P(self.mu), P(self.rstd), batch, self.C, ops._stream())


class PixelNorm(Module):
    """Pixel norm over C (no counterpart in the reference); eps = 1e-4 inside the root."""
    name = "pixel_norm"

    def __init__(self, C, pixels_per_sample=1, eps=1e-4):
        self.C, self.pps, self.eps = C, pixels_per_sample, eps
        self.in_dim = self.out_dim = C * pixels_per_sample

    def forward(self, inp, out, batch, ctx=None):
        ops._lib().launch_pixel_norm_forward(ops._p(out), ops._p(inp), batch * self.pps, self.C, self.eps, ops._stream())

    def backward(self, inp, out, grad_out, grad_in, batch, ctx=None):
        ops._lib().launch_pixel_norm_backward(ops._p(grad_in), ops._p(grad_out), ops._p(inp), batch * self.pps, self.C,
                                              self.eps, ops._stream())


class MPLinear(Module):
    """mp_linear_create(ctx, in_dim, out_dim, gain) -- src/mp_linear.c: the weight is normalised IN
    PLACE on every forward (eps 1e-4), the product goes to cuBLAS, the gain is a device scalar."""
    name = "mp_linear"

    def __init__(self, in_dim, out_dim, gain, device="cuda", generator=None):
        self.in_dim, self.out_dim, self.eps = in_dim, out_dim, 1e-4
        self.W = torch.randn(in_dim, out_dim, device=device, generator=generator)
        self.gW = torch.zeros_like(self.W)
        self.gain = torch.full((1,), float(gain), device=device)
        self.g_gain = torch.zeros(1, device=device)

    def forward(self, inp, out, batch, ctx=None):
        ops.weight_normalize_(self.W, self.eps)
        torch.matmul(inp.view(batch, self.in_dim), self.W, out=out.view(batch, self.out_dim))
        ops.scale_by_scalar_(out, self.gain)

    def backward(self, inp, out, grad_out, grad_in, batch, ctx=None):
        torch.matmul(inp.view(batch, self.in_dim).t(), grad_out.view(batch, self.out_dim), out=self.gW)
        self.g_gain.zero_()
        ops.weight_normalize_backward_(self.gW, self.W, self.gain, self.g_gain)
        if grad_in is not None:
            torch.matmul(grad_out.view(batch, self.out_dim), self.W.t(), out=grad_in.view(batch, self.in_dim))
            ops.scale_by_scalar_(grad_in, self.gain)

    def parameters(self, pl):
        pl.add(self.W, self.gW, self.W.numel())
        pl.add(self.gain, self.g_gain, 1)


class MPFourier(Module):
    """mp_fourier_create(ctx, num_channels, bandwidth) -- src/mp_fourier.c; no gradient flows back."""
    name = "mp_fourier"

    def __init__(self, num_channels, bandwidth, device="cuda", generator=None):
        self.in_dim, self.out_dim = 1, num_channels
        self.freqs = torch.randn(num_channels, device=device, generator=generator) * bandwidth
        self.phases = torch.rand(num_channels, device=device, generator=generator)

    def forward(self, inp, out, batch, ctx=None):
        P = ops._p
        ops._lib().launch_mp_fourier(P(out), P(inp), P(self.freqs), P(self.phases), batch, self.out_dim, ops._stream())

    def backward(self, inp, out, grad_out, grad_in, batch, ctx=None):
        pass  # fixed frequencies and a data-only input (src/mp_fourier.c:16-28): grad_in is left untouched


class Sinusoidal(Module):
    """sinusoidal_create(num_channels, max_period) -- src/sinusoidal.c; log(max_period) taken on the host."""
    name = "sinusoidal"

    def __init__(self, num_channels, max_period):
        if num_channels % 2:
            raise ValueError(f"sinusoidal_create: num_channels must be even (got {num_channels})")
        self.in_dim, self.out_dim = 1, num_channels
        self.log_max_period = math.log(max_period)

    def forward(self, inp, out, batch, ctx=None):
        ops._lib().launch_sinusoidal(ops._p(out), ops._p(inp), batch, self.out_dim, self.log_max_period, ops._stream())

    def backward(self, inp, out, grad_out, grad_in, batch, ctx=None):
        pass


# --------------------------------------------------------------------------- constructors (reference names)
def activation_create(dim, act):
    return Activation(dim, act)


def spatial_groupnorm_create(C, num_groups, H, W, max_batch, **kw):
    return SpatialGroupNorm(C, num_groups, H, W, max_batch, **kw)


def layernorm_create(dim, max_batch, **kw):
    return LayerNorm(dim, max_batch, **kw)


def mp_linear_create(ctx, in_dim, out_dim, gain, **kw):
    return MPLinear(in_dim, out_dim, gain, **kw)


def mp_fourier_create(ctx, num_channels, bandwidth, **kw):
    return MPFourier(num_channels, bandwidth, **kw)


def sinusoidal_create(num_channels, max_period):
    return Sinusoidal(num_channels, max_period)


# --------------------------------------------------------------------------- optimizer / EMA (src/optimizer.c, src/ema.c)
def _bias_correction(beta, t):
    return float(1.0 - torch.pow(torch.tensor(beta, dtype=torch.float32), torch.tensor(float(t), dtype=torch.float32)))


class Optimizer:
    """optimizer_adam(pl, lr, beta1, beta2, eps) / optimizer_step / optimizer_set_lr / timestep accessors."""

    def __init__(self, pl, lr, beta1, beta2, eps):
        self.lr, self.beta1, self.beta2, self.eps, self.t = lr, beta1, beta2, eps, 0
        self.m = [torch.zeros_like(it.param) for it in pl]
        self.v = [torch.zeros_like(it.param) for it in pl]

    def step(self, pl, ctx=None):
        """One launch per tensor, as optimizer.c:65-68."""
        self.t += 1
        bc1, bc2 = _bias_correction(self.beta1, self.t), _bias_correction(self.beta2, self.t)
        for it, m, v in zip(pl, self.m, self.v):
            ops.adam_step_(it.param, m, v, it.grad, self.lr, self.beta1, self.beta2, self.eps, bc1, bc2)

    def step_fused(self, pl, ema=None, grad_scale=1.0):
        """Adam for the whole list (and the EMA update when `ema` is given) in ONE launch."""
        self.t += 1
        bc1, bc2 = _bias_correction(self.beta1, self.t), _bias_correction(self.beta2, self.t)
        shadows = ema.shadow if ema is not None else [None] * len(pl)
        ops.adam_ema_step_multi_(((it.param, it.grad, m, v, sh) for it, m, v, sh in zip(pl, self.m, self.v, shadows)),
                                 self.lr, self.beta1, self.beta2, self.eps, bc1, bc2,
                                 ema.decay if ema is not None else 0.0, grad_scale)

    def set_lr(self, lr):
        self.lr = lr

    def timestep(self):
        return self.t

    def set_timestep(self, t):
        self.t = t

    def moment_lists(self):
        return list(self.m), list(self.v)


def optimizer_adam(pl, lr, beta1, beta2, eps):
    return Optimizer(pl, lr, beta1, beta2, eps)


class EMA:
    """ema_create(pl, decay) / ema_update / ema_swap -- src/ema.c"""

    def __init__(self, pl, decay):
        self.decay = decay
        self.shadow = [it.param.clone() for it in pl]

    def update(self, pl, ctx=None):
        one_minus = float(torch.tensor(1.0, dtype=torch.float32) - torch.tensor(self.decay, dtype=torch.float32))
        for sh, it in zip(self.shadow, pl):
            ops.weighted_sum(sh, it.param, self.decay, one_minus, out=sh)

    def swap(self, pl, ctx=None):
        for sh, it in zip(self.shadow, pl):
            tmp = it.param.clone()
            it.param.copy_(sh)
            sh.copy_(tmp)

    def shadow_list(self):
        return list(self.shadow)


def ema_create(pl, decay):
    return EMA(pl, decay)


def lr_inv_sqrt(lr_ref, step, t_warmup, t_ref):
    """src/nn.h:234-243"""
    warm = step / t_warmup if (t_warmup > 0 and step < t_warmup) else 1.0
    decay = math.sqrt(t_ref / step) if step > t_ref else 1.0
    return lr_ref * warm * decay
