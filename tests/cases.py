"""Shared parity cases: seeded inputs, and runners for the three implementations.

* `oracle_run`  -- the CPU oracle (oracle/layer_oracle.c), double accumulators.
* `gpu_run`     -- any CUDA library exporting the reference launcher set, called
                   through its C ABI: ours (fused entry points where they exist) or
                   the reference's own kernels built for sm_100a (composed calls).

Each case is (op, params); `make_inputs` derives every array from the case seed
with numpy's PCG64 generator, so the same inputs are rebuilt on any machine.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np

ACT = {"identity": 0, "relu": 1, "gelu": 2, "silu": 3, "tanh": 4, "mp_silu": 5}

# (name, op, params).  Small on purpose: the oracle runs each in milliseconds and
# the golden file stays a few hundred KB.
CASES = [
    ("act_silu", "act", dict(n=1031, act="silu")),
    ("act_mp_silu", "act", dict(n=4096, act="mp_silu")),
    ("act_gelu", "act", dict(n=777, act="gelu")),
    ("act_tanh", "act", dict(n=513, act="tanh")),
    ("act_relu", "act", dict(n=64, act="relu")),
    ("act_silu_wide", "act", dict(n=2048, act="silu", scale=6.0)),
    ("weighted_sum", "weighted_sum", dict(n=3001, wa=0.75, wb=-1.25)),
    ("mp_sum_t03", "mp_sum", dict(n=2048, t=0.3)),
    ("mp_cat_64_64", "mp_cat", dict(rows=37, Ca=64, Cb=64, t=0.5)),
    ("mp_cat_ragged", "mp_cat", dict(rows=19, Ca=6, Cb=9, t=0.3)),
    ("scale", "scale", dict(n=1000, s=0.37)),
    ("weight_norm_conv", "weight_norm", dict(rows=288, cols=32, eps=1e-4)),
    ("weight_norm_odd", "weight_norm", dict(rows=12, cols=6, eps=1e-4)),
    ("mp_fourier", "mp_fourier", dict(batch=16, C=128)),
    ("sinusoidal", "sinusoidal", dict(batch=16, C=64, max_period=1e4, tmax=50)),
    ("layernorm_256", "layernorm", dict(rows=33, C=256)),
    ("layernorm_16", "layernorm", dict(rows=5, C=16)),
    ("groupnorm_cfg0_small", "groupnorm", dict(B=3, HW=49, C=64, G=32, act=None)),
    ("groupnorm_gradcheck", "groupnorm", dict(B=2, HW=36, C=8, G=4, act=None)),
    ("groupnorm_silu", "groupnorm", dict(B=2, HW=64, C=32, G=4, act="silu")),
    ("groupnorm_odd", "groupnorm", dict(B=2, HW=15, C=6, G=3, act=None)),
    ("adam", "adam", dict(n=1500, steps=3)),
    ("adam_ema", "adam_ema", dict(n=1500, steps=3, decay=0.999)),
]


def seed_of(name):
    """Stable per-case seed (python's hash() is salted per process)."""
    return sum((i + 1) * ord(ch) for i, ch in enumerate(name)) % (2 ** 31)


def make_inputs(op, p, seed):
    rng = np.random.default_rng(seed)
    f = lambda *shape: rng.standard_normal(shape, dtype=np.float32)
    if op == "act":
        return dict(x=f(p["n"]) * np.float32(p.get("scale", 1.5)), g=f(p["n"]))
    if op in ("weighted_sum", "mp_sum"):
        return dict(a=f(p["n"]), b=f(p["n"]), g=f(p["n"]))
    if op == "mp_cat":
        return dict(a=f(p["rows"], p["Ca"]), b=f(p["rows"], p["Cb"]), g=f(p["rows"], p["Ca"] + p["Cb"]))
    if op == "scale":
        return dict(x=f(p["n"]), s=np.array([p["s"]], np.float32))
    if op == "weight_norm":
        return dict(W=f(p["rows"], p["cols"]), M=f(p["rows"], p["cols"]), gain=np.array([1.3], np.float32))
    if op == "mp_fourier":
        return dict(x=f(p["batch"]) * np.float32(0.5), freqs=f(p["C"]), phases=rng.random(p["C"], dtype=np.float32))
    if op == "sinusoidal":
        return dict(t=rng.integers(0, p["tmax"], p["batch"]).astype(np.float32))
    if op == "layernorm":
        C = p["C"]
        return dict(x=f(p["rows"], C), dy=f(p["rows"], C), gamma=1 + 0.1 * f(C), beta=0.1 * f(C))
    if op == "groupnorm":
        B, HW, C = p["B"], p["HW"], p["C"]
        return dict(x=f(B, HW, C), dy=f(B, HW, C), gamma=1 + 0.1 * f(C), beta=0.1 * f(C))
    if op == "pixel_norm":
        return dict(x=f(p["rows"], p["C"]), dy=f(p["rows"], p["C"]))
    if op in ("adam", "adam_ema"):
        n = p["n"]
        pr = (0.02 * f(n)).astype(np.float32)
        return dict(p=pr, g=[(1e-3 * f(n)).astype(np.float32) for _ in range(p["steps"])])
    raise KeyError(op)


ADAM = dict(lr=1e-4, b1=0.9, b2=0.999, eps=1e-8)


def _bias_corrections(t):
    # float32 powf as the reference host code does (optimizer.c:63-64)
    b1, b2 = np.float32(ADAM["b1"]), np.float32(ADAM["b2"])
    return float(np.float32(1) - np.power(b1, np.float32(t))), float(np.float32(1) - np.power(b2, np.float32(t)))


# --------------------------------------------------------------------------- oracle
def oracle_run(orc, op, p, inp):
    """orc: the imported oracle/oracle.py module.  Returns {name: ndarray}."""
    if op == "act":
        return dict(y=orc.activation_forward(inp["x"], p["act"]), gx=orc.activation_backward(inp["g"], inp["x"], p["act"]))
    if op == "weighted_sum":
        return dict(y=orc.weighted_sum(inp["a"], inp["b"], p["wa"], p["wb"]))
    if op == "mp_sum":
        ga, gb = orc.mp_sum_backward(inp["g"], p["t"])
        return dict(y=orc.mp_sum(inp["a"], inp["b"], p["t"]), ga=ga, gb=gb)
    if op == "mp_cat":
        ga, gb = orc.mp_channel_split(inp["g"], p["t"], p["Ca"], p["Cb"])
        return dict(y=orc.mp_cat(inp["a"], inp["b"], p["t"]), ga=ga, gb=gb)
    if op == "scale":
        return dict(y=orc.scale_by_scalar(inp["x"], inp["s"]))
    if op == "weight_norm":
        Wn = orc.weight_normalize(inp["W"], p["eps"])
        gW, gg = orc.weight_normalize_backward(inp["M"], Wn, float(inp["gain"][0]))
        return dict(Wn=Wn, gW=gW, g_gain=np.array([gg], np.float32))
    if op == "mp_fourier":
        return dict(y=orc.mp_fourier(inp["x"], inp["freqs"], inp["phases"]),
                    y64=orc.mp_fourier(inp["x"], inp["freqs"], inp["phases"], f64=True))
    if op == "sinusoidal":
        lmp = math.log(p["max_period"])
        return dict(y=orc.sinusoidal(inp["t"], p["C"], np.float32(lmp)),
                    y64=orc.sinusoidal(inp["t"], p["C"], np.float32(lmp), f64=True))
    if op == "layernorm":
        y, mu, rstd = orc.layernorm_forward(inp["x"], inp["gamma"], inp["beta"], 1e-5)
        dx, dg, db = orc.layernorm_backward(inp["dy"], inp["x"], inp["gamma"], mu, rstd)
        return dict(y=y, mu=mu, rstd=rstd, dx=dx, dgamma=dg, dbeta=db)
    if op == "groupnorm":
        y, mu, rstd = orc.groupnorm_forward(inp["x"], inp["gamma"], inp["beta"], p["G"], 1e-5, p["act"])
        dx, dg, db = orc.groupnorm_backward(inp["dy"], inp["x"], inp["gamma"], inp["beta"], mu, rstd, p["G"], p["act"])
        return dict(y=y, mu=mu, rstd=rstd, dx=dx, dgamma=dg, dbeta=db)
    if op == "pixel_norm":
        return dict(y=orc.pixel_norm_forward(inp["x"], p["eps"]), dx=orc.pixel_norm_backward(inp["dy"], inp["x"], p["eps"]))
    if op in ("adam", "adam_ema"):
        pr = inp["p"].copy(); m = np.zeros_like(pr); v = np.zeros_like(pr); sh = pr.copy()
        for t, g in enumerate(inp["g"], start=1):
            bc1, bc2 = _bias_corrections(t)
            if op == "adam":
                pr, m, v = orc.adam_step(pr, m, v, g, ADAM["lr"], ADAM["b1"], ADAM["b2"], ADAM["eps"], bc1, bc2)
            else:
                pr, m, v, sh = orc.adam_ema_step(pr, m, v, sh, g, ADAM["lr"], ADAM["b1"], ADAM["b2"], ADAM["eps"],
                                                 bc1, bc2, p["decay"])
        out = dict(p=pr, m=m, v=v)
        if op == "adam_ema":
            out["shadow"] = sh
        return out
    raise KeyError(op)


# --------------------------------------------------------------------------- GPU libraries
def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def gpu_run(lib, op, p, inp, fused, device_out=False):
    """Runs `op` through the C ABI of `lib` on cuda:0.  With fused=False only the
    reference launcher set is used (GroupNorm then activation, Adam then EMA as
    the reference's host code composes them).  Inputs may be host arrays or device
    tensors (never modified: in-place launchers work on a copy); with device_out the
    results stay on the device as tensors (the full-size cases compare there)."""
    import torch

    dev = torch.device("cuda:0")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def T(a):
        if isinstance(a, torch.Tensor):
            return a.to(dev, torch.float32).contiguous().clone()
        return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(dev)

    E = lambda *shape: torch.empty(*shape, device=dev, dtype=torch.float32)
    N = (lambda t: t) if device_out else (lambda t: t.cpu().numpy())
    F = ctypes.c_float

    if op == "act":
        x, g = T(inp["x"]), T(inp["g"]); y, gx = E(x.numel()), E(x.numel())
        lib.launch_activation_forward(_ptr(y), _ptr(x), x.numel(), ACT[p["act"]], st)
        lib.launch_activation_backward(_ptr(gx), _ptr(g), _ptr(x), x.numel(), ACT[p["act"]], st)
        return dict(y=N(y), gx=N(gx))
    if op == "weighted_sum":
        a, b = T(inp["a"]), T(inp["b"]); y = E(a.numel())
        lib.launch_weighted_sum(_ptr(y), _ptr(a), _ptr(b), F(p["wa"]), F(p["wb"]), a.numel(), st)
        return dict(y=N(y))
    if op == "mp_sum":
        a, b, g = T(inp["a"]), T(inp["b"]), T(inp["g"]); y, ga, gb = E(a.numel()), E(a.numel()), E(a.numel())
        lib.launch_mp_sum(_ptr(y), _ptr(a), _ptr(b), F(p["t"]), a.numel(), st)
        if fused:
            lib.launch_mp_sum_backward(_ptr(ga), _ptr(gb), _ptr(g), F(p["t"]), a.numel(), st)
        else:
            t = p["t"]; d = math.sqrt((1 - t) ** 2 + t ** 2)
            lib.launch_weighted_sum(_ptr(ga), _ptr(g), _ptr(g), F((1 - t) / d), F(0.0), a.numel(), st)
            lib.launch_weighted_sum(_ptr(gb), _ptr(g), _ptr(g), F(t / d), F(0.0), a.numel(), st)
        return dict(y=N(y), ga=N(ga), gb=N(gb))
    if op == "mp_cat":
        a, b, g = T(inp["a"]), T(inp["b"]), T(inp["g"])
        rows, Ca, Cb = p["rows"], p["Ca"], p["Cb"]
        y, ga, gb = E(rows, Ca + Cb), E(rows, Ca), E(rows, Cb)
        lib.launch_mp_channel_cat(_ptr(y), _ptr(a), _ptr(b), F(p["t"]), rows, Ca, Cb, st)
        lib.launch_mp_channel_split(_ptr(ga), _ptr(gb), _ptr(g), F(p["t"]), rows, Ca, Cb, st)
        y2 = E(rows, Ca + Cb)
        lib.launch_mp_cat(_ptr(y2), _ptr(a), _ptr(b), F(p["t"]), rows, Ca, Cb, st)
        assert torch.equal(y, y2), "launch_mp_cat and launch_mp_channel_cat disagree"
        return dict(y=N(y), ga=N(ga), gb=N(gb))
    if op == "scale":
        x, s = T(inp["x"]), T(inp["s"])
        lib.launch_scale_by_scalar(_ptr(x), _ptr(s), x.numel(), st)
        return dict(y=N(x))
    if op == "weight_norm":
        W, M, gain = T(inp["W"]), T(inp["M"]), T(inp["gain"]); gg = torch.zeros(1, device=dev)
        lib.launch_weight_normalize(_ptr(W), p["rows"], p["cols"], F(p["eps"]), st)
        lib.launch_weight_normalize_backward(_ptr(M), _ptr(W), _ptr(gain), _ptr(gg), p["rows"], p["cols"], st)
        return dict(Wn=N(W), gW=N(M), g_gain=N(gg))
    if op == "mp_fourier":
        x, fr, ph = T(inp["x"]), T(inp["freqs"]), T(inp["phases"]); y = E(p["batch"], p["C"])
        lib.launch_mp_fourier(_ptr(y), _ptr(x), _ptr(fr), _ptr(ph), p["batch"], p["C"], st)
        return dict(y=N(y))
    if op == "sinusoidal":
        t = T(inp["t"]); y = E(p["batch"], p["C"])
        lib.launch_sinusoidal(_ptr(y), _ptr(t), p["batch"], p["C"], F(np.float32(math.log(p["max_period"]))), st)
        return dict(y=N(y))
    if op == "layernorm":
        x, dy, ga, be = T(inp["x"]), T(inp["dy"]), T(inp["gamma"]), T(inp["beta"])
        rows, C = p["rows"], p["C"]
        y, mu, rstd, dx, dg, db = E(rows, C), E(rows), E(rows), E(rows, C), E(C), E(C)
        lib.launch_layernorm_forward(_ptr(y), _ptr(mu), _ptr(rstd), _ptr(x), _ptr(ga), _ptr(be), rows, C, F(1e-5), st)
        lib.launch_layernorm_backward(_ptr(dx), _ptr(dg), _ptr(db), _ptr(dy), _ptr(x), _ptr(ga), _ptr(mu), _ptr(rstd),
                                      rows, C, st)
        return dict(y=N(y), mu=N(mu), rstd=N(rstd), dx=N(dx), dgamma=N(dg), dbeta=N(db))
    if op == "groupnorm":
        x, dy, ga, be = T(inp["x"]), T(inp["dy"]), T(inp["gamma"]), T(inp["beta"])
        B, HW, C, G, act = p["B"], p["HW"], p["C"], p["G"], p["act"]
        y, mu, rstd, dx, dg, db = E(B, HW, C), E(B * G), E(B * G), E(B, HW, C), E(C), E(C)
        n = B * HW * C
        if act is None:
            lib.launch_groupnorm_forward(_ptr(y), _ptr(mu), _ptr(rstd), _ptr(x), _ptr(ga), _ptr(be), B, HW, C, G,
                                         F(1e-5), st)
            lib.launch_groupnorm_backward(_ptr(dx), _ptr(dg), _ptr(db), _ptr(dy), _ptr(x), _ptr(ga), _ptr(mu),
                                          _ptr(rstd), B, HW, C, G, st)
        elif fused:
            lib.launch_groupnorm_act_forward(_ptr(y), _ptr(mu), _ptr(rstd), _ptr(x), _ptr(ga), _ptr(be), B, HW, C, G,
                                             F(1e-5), ACT[act], st)
            lib.launch_groupnorm_act_backward(_ptr(dx), _ptr(dg), _ptr(db), _ptr(dy), _ptr(x), _ptr(ga), _ptr(be),
                                              _ptr(mu), _ptr(rstd), B, HW, C, G, ACT[act], st)
        else:
            h, gh = E(B, HW, C), E(B, HW, C)
            lib.launch_groupnorm_forward(_ptr(h), _ptr(mu), _ptr(rstd), _ptr(x), _ptr(ga), _ptr(be), B, HW, C, G,
                                         F(1e-5), st)
            lib.launch_activation_forward(_ptr(y), _ptr(h), n, ACT[act], st)
            lib.launch_activation_backward(_ptr(gh), _ptr(dy), _ptr(h), n, ACT[act], st)
            lib.launch_groupnorm_backward(_ptr(dx), _ptr(dg), _ptr(db), _ptr(gh), _ptr(x), _ptr(ga), _ptr(mu),
                                          _ptr(rstd), B, HW, C, G, st)
        return dict(y=N(y), mu=N(mu), rstd=N(rstd), dx=N(dx), dgamma=N(dg), dbeta=N(db))
    if op == "pixel_norm":
        x, dy = T(inp["x"]), T(inp["dy"]); rows, C = p["rows"], p["C"]
        y, dx = E(rows, C), E(rows, C)
        lib.launch_pixel_norm_forward(_ptr(y), _ptr(x), rows, C, F(p["eps"]), st)
        lib.launch_pixel_norm_backward(_ptr(dx), _ptr(dy), _ptr(x), rows, C, F(p["eps"]), st)
        return dict(y=N(y), dx=N(dx))
    if op in ("adam", "adam_ema"):
        pr = T(inp["p"]); m = torch.zeros_like(pr); v = torch.zeros_like(pr); sh = pr.clone()
        n = pr.numel()
        for t, g in enumerate(inp["g"], start=1):
            gt = T(g); bc1, bc2 = _bias_corrections(t)
            hp = (F(ADAM["lr"]), F(ADAM["b1"]), F(ADAM["b2"]), F(ADAM["eps"]), F(bc1), F(bc2))
            if op == "adam_ema" and fused:
                lib.launch_adam_ema_step(_ptr(pr), _ptr(m), _ptr(v), _ptr(sh), _ptr(gt), *hp, F(p["decay"]), F(1.0),
                                         ctypes.c_longlong(n), st)
            else:
                lib.launch_adam_step(_ptr(pr), _ptr(m), _ptr(v), _ptr(gt), *hp, n, st)
                if op == "adam_ema":
                    lib.launch_weighted_sum(_ptr(sh), _ptr(sh), _ptr(pr), F(p["decay"]), F(float(np.float32(1) - np.float32(p["decay"]))), n, st)
        torch.cuda.synchronize()
        out = dict(p=N(pr), m=N(m), v=N(v))
        if op == "adam_ema":
            out["shadow"] = N(sh)
        return out
    raise KeyError(op)


# --------------------------------------------------------------------------- comparison
# forward outputs: rel <= 1e-5, backward outputs: rel <= 1e-4 (the stated fp32 tolerance),
# both measured as max|a-b| / max(max|ref|, floor).
FWD_KEYS = {"y", "mu", "rstd", "Wn", "p", "m", "v", "shadow"}
TOL_FWD, TOL_BWD = 1e-5, 1e-4


def rel_err(a, ref, floor=1e-6):
    a = np.asarray(a, np.float64); ref = np.asarray(ref, np.float64)
    if a.size == 0:
        return 0.0
    return float(np.max(np.abs(a - ref)) / max(float(np.max(np.abs(ref))), floor))


def tolerance(key):
    return TOL_FWD if key in FWD_KEYS else TOL_BWD
