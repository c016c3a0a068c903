"""Tensor-level wrappers over the C ABI.

PyTorch is used for device memory and streams only: every function takes CUDA
fp32 tensors, passes their raw pointers and the current stream to the C entry
point, and returns tensors it allocated for the outputs.  Nothing here computes
on its own and nothing falls back to PyTorch or the CPU.
"""
from __future__ import annotations

import ctypes

import torch

from . import capi

ACT = {"identity": 0, "relu": 1, "gelu": 2, "silu": 3, "tanh": 4, "mp_silu": 5}


def _lib():
    return capi.load()


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    if t is None:
        return ctypes.c_void_p(0)
    assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous(), "expects contiguous CUDA fp32 tensors"
    return ctypes.c_void_p(t.data_ptr())


def _act(a):
    return ACT[a] if isinstance(a, str) else int(a)


# ----------------------------------------------------------------------------- element-wise
def activation_forward(x, act, out=None):
    out = torch.empty_like(x) if out is None else out
    _lib().launch_activation_forward(_p(out), _p(x), x.numel(), _act(act), _stream())
    return out


def activation_backward(grad_out, x, act, grad_in=None):
    grad_in = torch.empty_like(x) if grad_in is None else grad_in
    _lib().launch_activation_backward(_p(grad_in), _p(grad_out), _p(x), x.numel(), _act(act), _stream())
    return grad_in


def weighted_sum(a, b, wa, wb, out=None):
    out = torch.empty_like(a) if out is None else out
    _lib().launch_weighted_sum(_p(out), _p(a), _p(b), wa, wb, a.numel(), _stream())
    return out


def mp_sum(a, b, t, out=None):
    out = torch.empty_like(a) if out is None else out
    _lib().launch_mp_sum(_p(out), _p(a), _p(b), t, a.numel(), _stream())
    return out


def mp_sum_backward(g, t):
    ga, gb = torch.empty_like(g), torch.empty_like(g)
    _lib().launch_mp_sum_backward(_p(ga), _p(gb), _p(g), t, g.numel(), _stream())
    return ga, gb


def scale_by_scalar_(x, s):
    _lib().launch_scale_by_scalar(_p(x), _p(s), x.numel(), _stream())
    return x


def mp_cat(a, b, t):
    """a: [..., Ca], b: [..., Cb] (same leading shape) -> [..., Ca+Cb] scaled concat."""
    rows = a.numel() // a.shape[-1]
    out = torch.empty(*a.shape[:-1], a.shape[-1] + b.shape[-1], device=a.device, dtype=a.dtype)
    _lib().launch_mp_channel_cat(_p(out), _p(a), _p(b), t, rows, a.shape[-1], b.shape[-1], _stream())
    return out


def mp_cat_backward(g, t, Ca, Cb):
    rows = g.numel() // g.shape[-1]
    ga = torch.empty(*g.shape[:-1], Ca, device=g.device, dtype=g.dtype)
    gb = torch.empty(*g.shape[:-1], Cb, device=g.device, dtype=g.dtype)
    _lib().launch_mp_channel_split(_p(ga), _p(gb), _p(g), t, rows, Ca, Cb, _stream())
    return ga, gb


def axpby_rows(a, b, wa, wb, out=None):
    out = torch.empty_like(a) if out is None else out
    rows = a.shape[0]
    _lib().launch_axpby_rows(_p(out), _p(a), _p(b), _p(wa), _p(wb), rows, a.numel() // rows, _stream())
    return out


# ----------------------------------------------------------------------------- normalisation
def groupnorm_forward(x, gamma, beta, G, eps=1e-5, act=None):
    """x: [B, H, W, C] or [B, HW, C].  Returns (y, mu, rstd); act fuses an activation."""
    B, C = x.shape[0], x.shape[-1]
    HW = x.numel() // (B * C)
    y = torch.empty_like(x)
    mu = torch.empty(B * G, device=x.device, dtype=x.dtype)
    rstd = torch.empty_like(mu)
    if act is None:
        _lib().launch_groupnorm_forward(_p(y), _p(mu), _p(rstd), _p(x), _p(gamma), _p(beta), B, HW, C, G, eps,
                                        _stream())
    else:
        _lib().launch_groupnorm_act_forward(_p(y), _p(mu), _p(rstd), _p(x), _p(gamma), _p(beta), B, HW, C, G, eps,
                                            _act(act), _stream())
    return y, mu, rstd


def groupnorm_backward(dy, x, gamma, beta, mu, rstd, G, act=None):
    """Returns (dx, dgamma, dbeta)."""
    B, C = x.shape[0], x.shape[-1]
    HW = x.numel() // (B * C)
    dx = torch.empty_like(x)
    dgamma = torch.empty_like(gamma)
    dbeta = torch.empty_like(gamma)
    if act is None:
        _lib().launch_groupnorm_backward(_p(dx), _p(dgamma), _p(dbeta), _p(dy), _p(x), _p(gamma), _p(mu), _p(rstd),
                                         B, HW, C, G, _stream())
    else:
        _lib().launch_groupnorm_act_backward(_p(dx), _p(dgamma), _p(dbeta), _p(dy), _p(x), _p(gamma), _p(beta),
                                             _p(mu), _p(rstd), B, HW, C, G, _act(act), _stream())
    return dx, dgamma, dbeta


def layernorm_forward(x, gamma, beta, eps=1e-5):
    C = x.shape[-1]
    rows = x.numel() // C
    y = torch.empty_like(x)
    mu = torch.empty(rows, device=x.device, dtype=x.dtype)
    rstd = torch.empty_like(mu)
    _lib().launch_layernorm_forward(_p(y), _p(mu), _p(rstd), _p(x), _p(gamma), _p(beta), rows, C, eps, _stream())
    return y, mu, rstd


def layernorm_backward(dy, x, gamma, mu, rstd):
    C = x.shape[-1]
    rows = x.numel() // C
    dx = torch.empty_like(x)
    dgamma, dbeta = torch.empty_like(gamma), torch.empty_like(gamma)
    _lib().launch_layernorm_backward(_p(dx), _p(dgamma), _p(dbeta), _p(dy), _p(x), _p(gamma), _p(mu), _p(rstd),
                                     rows, C, _stream())
    return dx, dgamma, dbeta


def pixel_norm_forward(x, eps=1e-4):
    C = x.shape[-1]
    y = torch.empty_like(x)
    _lib().launch_pixel_norm_forward(_p(y), _p(x), x.numel() // C, C, eps, _stream())
    return y


def pixel_norm_backward(dy, x, eps=1e-4):
    C = x.shape[-1]
    dx = torch.empty_like(x)
    _lib().launch_pixel_norm_backward(_p(dx), _p(dy), _p(x), x.numel() // C, C, eps, _stream())
    return dx


# ----------------------------------------------------------------------------- weight norm
def weight_normalize_(W, eps=1e-4):
    """W: [in, out]; columns normalised in place."""
    _lib().launch_weight_normalize(_p(W), W.shape[0], W.shape[1], eps, _stream())
    return W


def weight_normalize_backward_(gW, Wn, gain, g_gain):
    """gW (holding M = x^T dZ) is overwritten with the tangent-projected gradient; g_gain is accumulated."""
    _lib().launch_weight_normalize_backward(_p(gW), _p(Wn), _p(gain), _p(g_gain), Wn.shape[0], Wn.shape[1],
                                            _stream())
    return gW


def weight_normalize_multi_(weights, eps=1e-4):
    arr = (capi.WeightDesc * len(weights))()
    for i, w in enumerate(weights):
        arr[i].W = w.data_ptr()
        arr[i].rows_in, arr[i].cols_out = w.shape
    _lib().launch_weight_normalize_multi(ctypes.cast(arr, ctypes.c_void_p), len(weights), eps, _stream())


# ----------------------------------------------------------------------------- embeddings
def mp_fourier(x, freqs, phases):
    out = torch.empty(x.numel(), freqs.numel(), device=x.device, dtype=x.dtype)
    _lib().launch_mp_fourier(_p(out), _p(x), _p(freqs), _p(phases), x.numel(), freqs.numel(), _stream())
    return out


def sinusoidal(t, C, log_max_period):
    out = torch.empty(t.numel(), C, device=t.device, dtype=t.dtype)
    _lib().launch_sinusoidal(_p(out), _p(t), t.numel(), C, log_max_period, _stream())
    return out


# ----------------------------------------------------------------------------- optimiser
def adam_step_(p, m, v, g, lr, b1, b2, eps, bc1, bc2):
    _lib().launch_adam_step(_p(p), _p(m), _p(v), _p(g), lr, b1, b2, eps, bc1, bc2, p.numel(), _stream())


def adam_ema_step_(p, m, v, shadow, g, lr, b1, b2, eps, bc1, bc2, decay, grad_scale=1.0):
    _lib().launch_adam_ema_step(_p(p), _p(m), _p(v), _p(shadow), _p(g), lr, b1, b2, eps, bc1, bc2, decay,
                                grad_scale, p.numel(), _stream())


def adam_ema_step_multi_(items, lr, b1, b2, eps, bc1, bc2, decay, grad_scale=1.0):
    """items: iterable of (p, g, m, v, shadow-or-None) tensors."""
    items = list(items)
    arr = (capi.ParamUpdate * len(items))()
    for i, (p, g, m, v, sh) in enumerate(items):
        arr[i].p, arr[i].g, arr[i].m, arr[i].v = p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr()
        arr[i].shadow = sh.data_ptr() if sh is not None else None
        arr[i].n = p.numel()
    _lib().launch_adam_ema_step_multi(ctypes.cast(arr, ctypes.c_void_p), len(items), lr, b1, b2, eps, bc1, bc2,
                                      decay, grad_scale, _stream())


# ----------------------------------------------------------------------------- management
def launch_count():
    return int(_lib().b200_launch_count())


def tune_set(key, value):
    _lib().b200_tune_set(key.encode(), int(value))


def set_error_mode(mode):
    _lib().b200_set_error_mode(int(mode))


def last_error():
    buf = ctypes.create_string_buffer(1024)
    _lib().b200_last_error(ctypes.cast(buf, ctypes.c_void_p), 1024)
    return buf.value.decode()


def error_count():
    return int(_lib().b200_error_count())


def clear_error():
    _lib().b200_clear_error()


def device_error_status():
    return int(_lib().b200_device_error_status())
