"""GPU: element-wise A/B parity at the FULL benchmark configurations.

Every op of the five benchmark configurations runs through this library's C ABI (the fused
entry points where they exist) and through the reference's own kernels.cu built for sm_100a
(composed the way the reference's host code composes them), on the same seeded device inputs,
and every output tensor is compared element by element: forward rel <= 1e-5, backward
rel <= 1e-4 (max|a-b| / max|ref|, cases.TOL_FWD / TOL_BWD).  The normalisation layers are compared
three ways, with an fp64 evaluation as arbiter, because the reference's own kernels are racy at these
sizes (see _norm_three_way).  The embeddings are judged against
an fp64 evaluation with an absolute bound proportional to the argument's fp32 rounding, and the
reference's own error against the same truth is printed beside ours.

The reference's parameter-gradient kernels are serial per channel, so its side of a case takes
tens of milliseconds; the whole file runs in well under a minute.
"""
import math

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu


def _gen(seed):
    import torch
    return torch.Generator(device="cuda").manual_seed(seed)


def _randn(g, *shape):
    import torch
    return torch.randn(*shape, device="cuda", generator=g)


def _rel(a, ref):
    return float((a.double() - ref.double()).abs().max()) / max(float(ref.abs().max()), 1e-6)


def _ab(lib, ref_lib, op, p, inp, label, skip=()):
    import torch
    got = cases.gpu_run(lib, op, p, inp, fused=True, device_out=True)
    ref = cases.gpu_run(ref_lib, op, p, inp, fused=False, device_out=True)
    torch.cuda.synchronize()
    worst = {}
    for k, r in ref.items():
        if k in skip:
            continue
        e = _rel(got[k], r)
        worst[k] = e
        assert e <= cases.tolerance(k), f"{label}:{k} rel err {e:.3e} > {cases.tolerance(k):.0e}"
    print(label, {k: f"{v:.1e}" for k, v in worst.items()})
    del got, ref
    torch.cuda.empty_cache()


def _norm_inputs(g, B, HW, C):
    return dict(x=_randn(g, B, HW, C), dy=_randn(g, B, HW, C), gamma=1 + 0.1 * _randn(g, C), beta=0.1 * _randn(g, C))


# ---- normalisation layers: three-way comparison -------------------------------------------------
# The reference's GroupNorm / LayerNorm kernels call block_reduce_sum twice in a row
# (src/kernels.cu:72-91 used at :647-648, :681-682, :505-512, :535-540).  The second call's first
# shared-memory write is not separated by a barrier from the first call's final read, so a warp that
# is late reads the wrong total and normalises its elements with it.  On a B200 at these grid sizes
# that happens in a small share of the blocks (the statistics mu/rstd, written by thread 0, stay
# right).  An element-wise A/B therefore needs an arbiter: an fp64 evaluation of the same formulas
# on the device.  Every output must match the fp64 truth to the stated tolerance; it must match the
# reference's kernels to the same tolerance in every (sample, group) / row that the reference's
# race did not hit; and the share of hit units is printed and bounded.
def _rational_sigmoid64(z):
    h = 0.5 * z
    h2 = h * h
    num = h * (135135.0 + h2 * (17325.0 + h2 * (378.0 + h2)))
    den = 135135.0 + h2 * (62370.0 + h2 * (3150.0 + h2 * 28.0))
    return ((num / den).clamp(-1.0, 1.0) + 1.0) * 0.5


def _norm_truth(inp, B, HW, C, G, act):
    """fp64 GroupNorm (+SiLU as the reference's rational form, kernels.cu:6-17,49-56) forward and backward;
    LayerNorm is the case G=1 over a [rows,1,C] view."""
    x = inp["x"].double().view(B, HW, G, C // G)
    dy = inp["dy"].double().view(B, HW, C)
    ga, be = inp["gamma"].double(), inp["beta"].double()
    mu = x.mean(dim=(1, 3))
    rstd = (x.var(dim=(1, 3), unbiased=False) + 1e-5).rsqrt()
    xh = ((x - mu[:, None, :, None]) * rstd[:, None, :, None]).view(B, HW, C)
    z = xh * ga + be
    if act == "silu":
        sg = _rational_sigmoid64(z)
        y = z * sg
        gz = dy * (sg * (1.0 + z * (1.0 - sg)))
        del sg
    else:
        y, gz = z, dy
    del z
    dgamma, dbeta = (gz * xh).sum(dim=(0, 1)), gz.sum(dim=(0, 1))
    gg = (gz * ga).view(B, HW, G, C // G)
    del gz
    m1 = gg.mean(dim=(1, 3))
    m2 = (gg * xh.view(B, HW, G, C // G)).mean(dim=(1, 3))
    dx = (rstd[:, None, :, None] * (gg - m1[:, None, :, None] - xh.view(B, HW, G, C // G) * m2[:, None, :, None])).view(B, HW, C)
    return dict(y=y, mu=mu.reshape(-1), rstd=rstd.reshape(-1), dx=dx, dgamma=dgamma, dbeta=dbeta)


def _norm_three_way(lib, ref_lib, op, p, inp, shape, label):
    import torch
    B, HW, C, G, act = shape
    got = cases.gpu_run(lib, op, p, inp, fused=True, device_out=True)
    ref = cases.gpu_run(ref_lib, op, p, inp, fused=False, device_out=True)
    truth = _norm_truth(inp, B, HW, C, G, act)
    torch.cuda.synchronize()
    report, fwd_hits = {}, 0
    for k, t in truth.items():
        tol = cases.tolerance(k)
        scale = max(float(t.abs().max()), 1e-6)
        e_truth = float((got[k].double().view_as(t) - t).abs().max()) / scale
        assert e_truth <= tol, f"{label}:{k} vs fp64 truth: rel err {e_truth:.3e} > {tol:.0e}"
        d_ref = (ref[k].double().view_as(t) - t).abs()
        d_ab = (got[k].double() - ref[k].double()).abs().view_as(t)
        if k in ("y", "dx"):
            # a unit = one (sample, group) / one row; "hit" = the reference itself is further than half the
            # tolerance from the truth there (this library is within ~1e-6 of it everywhere)
            unit = lambda e: e.view(B, HW, G, C // G).amax(dim=(1, 3))
            hit = unit(d_ref) > 0.5 * tol * scale
            n_hit, n_units = int(hit.sum()), hit.numel()
            if k == "y":
                fwd_hits = n_hit
            assert n_hit <= 0.1 * n_units, f"{label}:{k}: the reference is off in {n_hit} of {n_units} units"
            e_ab = float(unit(d_ab)[~hit].max()) / scale
            report[k] = (f"truth {e_truth:.1e}, A/B {e_ab:.1e} outside the {n_hit}/{n_units} units where the "
                         f"reference's race struck (its worst error there {float(d_ref.max()) / scale:.1e})")
            assert e_ab <= tol, f"{label}:{k} vs reference kernels: rel err {e_ab:.3e} > {tol:.0e}"
        else:
            e_ab = float(d_ab.max()) / scale
            report[k] = f"truth {e_truth:.1e}, A/B {e_ab:.1e}"
            # with a fused activation the reference's parameter gradients are sums over its own activation
            # gradient, which inherits the forward's race; they are only comparable when no unit was hit
            if k in ("dgamma", "dbeta") and act is not None and fwd_hits > 0:
                report[k] += " (not asserted: the reference's sums include race-hit units)"
            else:
                assert e_ab <= tol, f"{label}:{k} vs reference kernels: rel err {e_ab:.3e} > {tol:.0e}"
        del d_ref, d_ab
    print(label, report)
    del got, ref, truth
    torch.cuda.empty_cache()


def test_groupnorm_128x28x28x64(lib, ref_lib):
    """Configuration 1: GroupNorm forward+backward, [128,28,28,64], 32 groups, eps 1e-5, seed 0."""
    p = dict(B=128, HW=784, C=64, G=32, act=None)
    _norm_three_way(lib, ref_lib, "groupnorm", p, _norm_inputs(_gen(0), 128, 784, 64), (128, 784, 64, 32, None),
                    "cfg1/groupnorm")


def test_edm_op_set_256x28x28x128(lib, ref_lib):
    """Configuration 2: MP-SiLU, mp_sum(t=0.3), mp_cat of two 64-channel tensors (t=0.5) and the forced
    weight normalisation of a [1152,128] weight, forward and backward.  (Pixel norm has no reference
    implementation; it is checked against the oracle and by its invariants elsewhere.)"""
    g = _gen(1)
    n = 256 * 28 * 28 * 128
    rows = 256 * 28 * 28
    _ab(lib, ref_lib, "act", dict(n=n, act="mp_silu"), dict(x=_randn(g, n), g=_randn(g, n)), "cfg2/mp_silu")
    _ab(lib, ref_lib, "act", dict(n=n, act="silu"), dict(x=_randn(g, n), g=_randn(g, n)), "cfg2/silu")
    _ab(lib, ref_lib, "mp_sum", dict(n=n, t=0.3), dict(a=_randn(g, n), b=_randn(g, n), g=_randn(g, n)), "cfg2/mp_sum")
    _ab(lib, ref_lib, "mp_cat", dict(rows=rows, Ca=64, Cb=64, t=0.5),
        dict(a=_randn(g, rows, 64), b=_randn(g, rows, 64), g=_randn(g, rows, 128)), "cfg2/mp_cat")
    import torch
    wn = dict(W=_randn(g, 1152, 128), M=_randn(g, 1152, 128), gain=torch.ones(1, device="cuda"))
    _ab(lib, ref_lib, "weight_norm", dict(rows=1152, cols=128, eps=1e-4), wn, "cfg2/weight_norm")


@pytest.mark.parametrize("rows,cols", [(2304, 128), (2304, 256), (3072, 64), (3080, 64), (576, 1), (576, 3), (27, 8)])
def test_weight_norm_shapes_of_the_unets(lib, ref_lib, rows, cols):
    """Weights beyond the benchmark's [1152,128]: 3x3 convolutions over 256 input channels (cluster kernel with 9-12
    register slots per thread), one row more than the cluster kernel holds (strip kernel), and the narrow
    matrices of a UNet's last convolution (one CTA per column)."""
    import torch
    g = _gen(7)
    wn = dict(W=_randn(g, rows, cols), M=_randn(g, rows, cols), gain=torch.full((1,), 1.3, device="cuda"))
    _ab(lib, ref_lib, "weight_norm", dict(rows=rows, cols=cols, eps=1e-4), wn, f"weight_norm[{rows},{cols}]")


def test_ddpm_block_kernels_256x32x32x256(lib, ref_lib):
    """Configuration 3: GroupNorm(32)+affine+SiLU (fused here; GroupNorm then SiLU in the reference, as
    conv_residual.c:28-29,51-52 composes them) and LayerNorm over C=256 on the same tensor viewed as
    [262144,256] tokens."""
    g = _gen(2)
    inp = _norm_inputs(g, 256, 1024, 256)
    _norm_three_way(lib, ref_lib, "groupnorm", dict(B=256, HW=1024, C=256, G=32, act="silu"), inp,
                    (256, 1024, 256, 32, "silu"), "cfg3/groupnorm_silu")
    _norm_three_way(lib, ref_lib, "groupnorm", dict(B=256, HW=1024, C=256, G=32, act=None), inp,
                    (256, 1024, 256, 32, None), "cfg3/groupnorm")
    ln = dict(x=inp["x"].view(262144, 256), dy=inp["dy"].view(262144, 256), gamma=inp["gamma"], beta=inp["beta"])
    _norm_three_way(lib, ref_lib, "layernorm", dict(rows=262144, C=256), ln, (262144, 1, 256, 1, None), "cfg3/layernorm")


def _embedding_errors(lib, ref_fast, ref_precise, op, p, inp, truth, bound, label):
    ours = cases.gpu_run(lib, op, p, inp, fused=True)["y"].astype(np.float64)
    e_ours = float(np.max(np.abs(ours - truth)))
    e_prec = float(np.max(np.abs(cases.gpu_run(ref_precise, op, p, inp, fused=False)["y"].astype(np.float64) - truth)))
    e_fast = float(np.max(np.abs(cases.gpu_run(ref_fast, op, p, inp, fused=False)["y"].astype(np.float64) - truth)))
    print(f"{label}: max abs error vs fp64 -- this library {e_ours:.2e}, reference without fast-math {e_prec:.2e}, "
          f"reference as shipped (--use_fast_math) {e_fast:.2e}; bound {bound:.2e}")
    assert e_ours <= bound, f"{label}: abs err {e_ours:.3e} > {bound:.3e}"
    return e_ours, e_prec, e_fast


def test_sinusoidal_embedding_dim512_t_below_1000(lib, orc, ref_lib, ref_lib_precise):
    """Configuration 3: integer timesteps t ~ U[0,1000) as floats, dim 512, max period 1e4.  sin(t*f) at
    t ~ 1000 amplifies the fp32 rounding of the argument (t*f*2^-24) into the output, so the tolerance is
    absolute: 4*tmax*2^-23 + 2e-6."""
    rng = np.random.default_rng(3)
    t = rng.integers(0, 1000, 256).astype(np.float32)
    t[:2] = (0.0, 999.0)
    p = dict(batch=256, C=512, max_period=1e4, tmax=1000)
    truth = orc.sinusoidal(t, 512, np.float32(math.log(1e4)), f64=True)
    bound = 4.0 * 1000 * 2.0 ** -23 + 2e-6
    _embedding_errors(lib, ref_lib, ref_lib_precise, "sinusoidal", p, dict(t=t), truth, bound, "cfg3/sinusoidal")


def test_mp_fourier_embedding_256_to_128(lib, orc, ref_lib, ref_lib_precise):
    """Configuration 4's noise-level embedding: x[256] -> [256,128], frequencies ~ N(0,1), phases ~ U[0,1);
    x = ln(sigma)/4 with sigma log-normal(P_mean -1.2, P_std 1.2) as diffusion/edm.c draws it."""
    rng = np.random.default_rng(4)
    x = ((-1.2 + 1.2 * rng.standard_normal(256)) / 4).astype(np.float32)
    inp = dict(x=x, freqs=rng.standard_normal(128).astype(np.float32), phases=rng.random(128, dtype=np.float32))
    truth = orc.mp_fourier(inp["x"], inp["freqs"], inp["phases"], f64=True)
    amax = 2 * math.pi * (float(np.abs(x).max()) * float(np.abs(inp["freqs"]).max()) + 1.0)
    bound = math.sqrt(2) * 4.0 * amax * 2.0 ** -23 + 2e-6
    _embedding_errors(lib, ref_lib, ref_lib_precise, "mp_fourier", dict(batch=256, C=128), inp, truth, bound,
                      "cfg4/mp_fourier")


def test_adam_then_ema_64M_params_three_steps(lib, ref_lib):
    """Configuration 5: flat vector of 64M parameters ~ N(0,0.02), gradients ~ N(0,1e-3); this library's one
    fused Adam+EMA pass against the reference's adam_step followed by its EMA weighted_sum, t = 1..3."""
    g = _gen(5)
    n = 64 * 2 ** 20
    inp = dict(p=0.02 * _randn(g, n), g=[1e-3 * _randn(g, n) for _ in range(3)])
    _ab(lib, ref_lib, "adam_ema", dict(n=n, steps=3, decay=0.999), inp, "cfg5/adam_ema")
    _ab(lib, ref_lib, "adam", dict(n=n, steps=3), inp, "cfg5/adam")
