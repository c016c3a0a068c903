"""numpy-facing binding of the CPU oracle (liblayer_oracle.so) -- TEST INFRASTRUCTURE.

Only tests/, the smoke check and the benchmark's CPU-baseline leg import this.
`load()` builds the shared object with gcc when it is missing or stale.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SO = HERE / "liblayer_oracle.so"
SRC = HERE / "layer_oracle.c"
HDR = HERE / "layer_oracle.h"

ACT = {"identity": 0, "relu": 1, "gelu": 2, "silu": 3, "tanh": 4, "mp_silu": 5}

_lib = None


def build(force: bool = False) -> Path:
    stale = (not SO.exists()) or SO.stat().st_mtime < max(SRC.stat().st_mtime, HDR.stat().st_mtime)
    if force or stale:
        subprocess.run(["gcc", "-O3", "-std=c11", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
                        str(SRC), "-o", str(SO), "-lm"], check=True)
    return SO


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.oracle_act_apply.restype = ctypes.c_float
        _lib.oracle_act_apply.argtypes = [ctypes.c_float, ctypes.c_int]
        _lib.oracle_act_grad.restype = ctypes.c_float
        _lib.oracle_act_grad.argtypes = [ctypes.c_float, ctypes.c_int]
        _lib.oracle_max_threads.restype = ctypes.c_int
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _call(name, *args):
    """Calls oracle_<name>; numpy arrays go as pointers, python ints as c_long/c_int by position table."""
    fn = getattr(load(), "oracle_" + name)
    conv = []
    for a in args:
        if isinstance(a, np.ndarray):
            conv.append(_ptr(a))
        elif isinstance(a, float):
            conv.append(ctypes.c_float(a))
        elif isinstance(a, L):
            conv.append(ctypes.c_long(int(a)))
        elif isinstance(a, (int, np.integer)):
            conv.append(ctypes.c_int(int(a)))
        else:
            raise TypeError(type(a))
    fn(*conv)


class L(int):
    """marks an argument that the C prototype declares as `long`"""


def set_accumulate_double(on: bool):
    load().oracle_set_accumulate_double(ctypes.c_int(1 if on else 0))


def set_threads(n: int):
    load().oracle_set_threads(ctypes.c_int(int(n)))


def max_threads() -> int:
    return int(load().oracle_max_threads())


def act_id(a):
    return ACT[a] if isinstance(a, str) else int(a)


# ---------------------------------------------------------------- element-wise
def activation_forward(x, act):
    x = _f(x); out = np.empty_like(x)
    _call("activation_forward", out, x, L(x.size), act_id(act))
    return out


def activation_backward(gout, x, act):
    x = _f(x); gout = _f(gout); out = np.empty_like(x)
    _call("activation_backward", out, gout, x, L(x.size), act_id(act))
    return out


def weighted_sum(a, b, wa, wb):
    a = _f(a); b = _f(b); out = np.empty_like(a)
    _call("weighted_sum", out, a, b, float(wa), float(wb), L(a.size))
    return out


def mp_sum(a, b, t):
    a = _f(a); b = _f(b); out = np.empty_like(a)
    _call("mp_sum", out, a, b, float(t), L(a.size))
    return out


def mp_sum_backward(g, t):
    g = _f(g); ga = np.empty_like(g); gb = np.empty_like(g)
    _call("mp_sum_backward", ga, gb, g, float(t), L(g.size))
    return ga, gb


def mp_cat(a, b, t):
    a = _f(a); b = _f(b)
    rows = a.size // a.shape[-1]
    out = np.empty(a.shape[:-1] + (a.shape[-1] + b.shape[-1],), np.float32)
    _call("mp_cat", out, a, b, float(t), L(rows), a.shape[-1], b.shape[-1])
    return out


def mp_channel_split(g, t, Ca, Cb):
    g = _f(g)
    rows = g.size // g.shape[-1]
    ga = np.empty(g.shape[:-1] + (Ca,), np.float32); gb = np.empty(g.shape[:-1] + (Cb,), np.float32)
    _call("mp_channel_split", ga, gb, g, float(t), L(rows), Ca, Cb)
    return ga, gb


def channel_cat(a, b):
    a = _f(a); b = _f(b)
    out = np.empty(a.shape[:-1] + (a.shape[-1] + b.shape[-1],), np.float32)
    _call("channel_cat", out, a, b, L(a.size // a.shape[-1]), a.shape[-1], b.shape[-1])
    return out


def channel_split(g, Ca, Cb):
    g = _f(g)
    ga = np.empty(g.shape[:-1] + (Ca,), np.float32); gb = np.empty(g.shape[:-1] + (Cb,), np.float32)
    _call("channel_split", ga, gb, g, L(g.size // g.shape[-1]), Ca, Cb)
    return ga, gb


def scale_by_scalar(x, s):
    x = _f(x).copy(); s = _f(s)
    _call("scale_by_scalar", x, s, L(x.size))
    return x


def axpby_rows(a, b, wa, wb):
    a = _f(a); b = _f(b); wa = _f(wa); wb = _f(wb); out = np.empty_like(a)
    _call("axpby_rows", out, a, b, wa, wb, a.shape[0], a.size // a.shape[0])
    return out


# ---------------------------------------------------------------- weight norm
def weight_normalize(W, eps):
    W = _f(W).copy()
    _call("weight_normalize", W, W.shape[0], W.shape[1], float(eps))
    return W


def weight_normalize_backward(gW, Wn, gain, g_gain0=0.0):
    gW = _f(gW).copy(); Wn = _f(Wn)
    gain = _f(np.array([gain])); gg = _f(np.array([g_gain0]))
    _call("weight_normalize_backward", gW, Wn, gain, gg, Wn.shape[0], Wn.shape[1])
    return gW, float(gg[0])


# ---------------------------------------------------------------- embeddings
def mp_fourier(x, freqs, phases, f64=False):
    x = _f(x); freqs = _f(freqs); phases = _f(phases)
    out = np.empty((x.size, freqs.size), np.float64 if f64 else np.float32)
    _call("mp_fourier_f64" if f64 else "mp_fourier", out, x, freqs, phases, x.size, freqs.size)
    return out


def sinusoidal(t, C, log_max_period, f64=False):
    t = _f(t)
    out = np.empty((t.size, C), np.float64 if f64 else np.float32)
    _call("sinusoidal_f64" if f64 else "sinusoidal", out, t, t.size, C, float(log_max_period))
    return out


# ---------------------------------------------------------------- normalisation
def layernorm_forward(x, gamma, beta, eps):
    x = _f(x); C = x.shape[-1]; rows = x.size // C
    y = np.empty_like(x); mu = np.empty(rows, np.float32); rstd = np.empty(rows, np.float32)
    _call("layernorm_forward", y, mu, rstd, x, _f(gamma), _f(beta), L(rows), C, float(eps))
    return y, mu, rstd


def layernorm_backward(dy, x, gamma, mu, rstd):
    x = _f(x); C = x.shape[-1]; rows = x.size // C
    dx = np.empty_like(x); dg = np.empty(C, np.float32); db = np.empty(C, np.float32)
    _call("layernorm_backward", dx, dg, db, _f(dy), x, _f(gamma), _f(mu), _f(rstd), L(rows), C)
    return dx, dg, db


def groupnorm_forward(x, gamma, beta, G, eps, act=None):
    x = _f(x); B, C = x.shape[0], x.shape[-1]; HW = x.size // (B * C)
    y = np.empty_like(x); mu = np.empty(B * G, np.float32); rstd = np.empty(B * G, np.float32)
    if act is None:
        _call("groupnorm_forward", y, mu, rstd, x, _f(gamma), _f(beta), B, HW, C, G, float(eps))
    else:
        _call("groupnorm_act_forward", y, mu, rstd, x, _f(gamma), _f(beta), B, HW, C, G, float(eps), act_id(act))
    return y, mu, rstd


def groupnorm_backward(dy, x, gamma, beta, mu, rstd, G, act=None):
    x = _f(x); B, C = x.shape[0], x.shape[-1]; HW = x.size // (B * C)
    dx = np.empty_like(x); dg = np.empty(C, np.float32); db = np.empty(C, np.float32)
    if act is None:
        _call("groupnorm_backward", dx, dg, db, _f(dy), x, _f(gamma), _f(mu), _f(rstd), B, HW, C, G)
    else:
        _call("groupnorm_act_backward", dx, dg, db, _f(dy), x, _f(gamma), _f(beta), _f(mu), _f(rstd), B, HW, C, G,
              act_id(act))
    return dx, dg, db


def pixel_norm_forward(x, eps):
    x = _f(x); C = x.shape[-1]; y = np.empty_like(x)
    _call("pixel_norm_forward", y, x, L(x.size // C), C, float(eps))
    return y


def pixel_norm_backward(dy, x, eps):
    x = _f(x); C = x.shape[-1]; dx = np.empty_like(x)
    _call("pixel_norm_backward", dx, _f(dy), x, L(x.size // C), C, float(eps))
    return dx


# ---------------------------------------------------------------- optimiser
def adam_step(p, m, v, g, lr, b1, b2, eps, bc1, bc2):
    p = _f(p).copy(); m = _f(m).copy(); v = _f(v).copy()
    _call("adam_step", p, m, v, _f(g), float(lr), float(b1), float(b2), float(eps), float(bc1), float(bc2), L(p.size))
    return p, m, v


def adam_ema_step(p, m, v, shadow, g, lr, b1, b2, eps, bc1, bc2, decay, grad_scale=1.0):
    p = _f(p).copy(); m = _f(m).copy(); v = _f(v).copy(); shadow = _f(shadow).copy()
    _call("adam_ema_step", p, m, v, shadow, _f(g), float(lr), float(b1), float(b2), float(eps), float(bc1),
          float(bc2), float(decay), float(grad_scale), L(p.size))
    return p, m, v, shadow


def raw(name, *args):
    """Direct access for the remaining launchers (see layer_oracle.h for the argument order)."""
    _call(name, *args)
