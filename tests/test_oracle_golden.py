"""CPU: the plain-C oracle against golden outputs of the reference's own CUDA kernels
(tests/golden/reference_kernels.npz, produced by tests/golden/make_golden.py on a B200), plus
independent closed-form checks of the oracle in numpy."""
from pathlib import Path

import numpy as np
import pytest

import cases

GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_kernels.npz"


@pytest.fixture(scope="module")
def golden():
    if not GOLDEN.exists():
        pytest.skip("golden file not generated yet")
    return np.load(GOLDEN)


@pytest.mark.parametrize("name,op,p", cases.CASES, ids=[c[0] for c in cases.CASES])
def test_oracle_matches_reference_kernel_outputs(orc, golden, name, op, p):
    inp = cases.make_inputs(op, p, seed=cases.seed_of(name))
    flat = np.concatenate([np.ravel(np.concatenate(v) if isinstance(v, list) else v).astype(np.float64)
                           for v in inp.values()])
    assert np.allclose(golden[f"{name}/__input_sum"], [flat.sum(), np.abs(flat).sum()], rtol=1e-12), \
        "seeded inputs differ from the ones the golden file was generated with"
    got = cases.oracle_run(orc, op, p, inp)
    for k, v in got.items():
        if k == "y64":
            continue
        ref = golden[f"{name}/{k}"]
        if op in ("mp_fourier", "sinusoidal"):
            tmax = p.get("tmax", 8 * np.pi)
            tol = 8.0 * max(tmax, 1.0) * 2.0 ** -23 + 4e-6
            assert float(np.max(np.abs(v.astype(np.float64) - ref))) <= tol, f"{name}:{k}"
        else:
            e = cases.rel_err(v, ref)
            assert e <= cases.tolerance(k), f"{name}:{k} rel err {e:.3e}"


def test_rational_tanh_is_the_reference_approximation(orc):
    """Closed form of kernels.cu:6-12 evaluated independently in float64."""
    x = np.linspace(-12, 12, 4801).astype(np.float32)
    x2 = x.astype(np.float64) ** 2
    num = x * (135135.0 + x2 * (17325.0 + x2 * (378.0 + x2)))
    den = 135135.0 + x2 * (62370.0 + x2 * (3150.0 + x2 * 28.0))
    ref = np.clip(num / den, -1.0, 1.0)
    got = orc.activation_forward(x, "tanh")
    assert np.max(np.abs(got - ref)) < 5e-7  # fp32 evaluation vs float64
    # it is an approximation: close to tanh for |x| < 4, clamped beyond ~4.97
    assert np.max(np.abs(ref - np.tanh(x))) < 1.2e-4
    sil = orc.activation_forward(x, "silu")
    assert np.max(np.abs(sil - x * (ref_half(x) + 1) / 2)) < 4e-6  # inputs up to 12 in fp32
    mps = orc.activation_forward(x, "mp_silu")
    assert np.allclose(mps, sil * np.float32(1.0 / 0.596), rtol=1e-6, atol=1e-7)


def ref_half(x):
    h = x.astype(np.float64) * 0.5
    h2 = h * h
    num = h * (135135.0 + h2 * (17325.0 + h2 * (378.0 + h2)))
    den = 135135.0 + h2 * (62370.0 + h2 * (3150.0 + h2 * 28.0))
    return np.clip(num / den, -1.0, 1.0)


def test_norm_oracles_against_numpy(orc):
    rng = np.random.default_rng(3)
    B, HW, C, G = 3, 10, 12, 3
    x = rng.standard_normal((B, HW, C)).astype(np.float32) * 2 + 1
    gam = rng.standard_normal(C).astype(np.float32); bet = rng.standard_normal(C).astype(np.float32)
    y, mu, rstd = orc.groupnorm_forward(x, gam, bet, G, 1e-5)
    xg = x.astype(np.float64).reshape(B, HW, G, C // G)
    m = xg.mean(axis=(1, 3), keepdims=True); v = xg.var(axis=(1, 3), keepdims=True)
    ref = ((xg - m) / np.sqrt(v + 1e-5)).reshape(B, HW, C) * gam + bet
    assert np.max(np.abs(y - ref)) < 1e-5
    assert np.allclose(mu, m.reshape(-1), atol=1e-6) and np.allclose(rstd, 1 / np.sqrt(v.reshape(-1) + 1e-5), rtol=1e-6)
    # backward: directional derivative check of dx in float64
    dy = rng.standard_normal((B, HW, C)).astype(np.float32)
    dx, dg, db = orc.groupnorm_backward(dy, x, gam, bet, mu, rstd, G)

    def f(xx):
        g_ = xx.reshape(B, HW, G, C // G)
        mm = g_.mean(axis=(1, 3), keepdims=True); vv = g_.var(axis=(1, 3), keepdims=True)
        return (((g_ - mm) / np.sqrt(vv + 1e-5)).reshape(B, HW, C) * gam + bet) * dy
    d = rng.standard_normal((B, HW, C))
    eps = 1e-6
    num = (f(x.astype(np.float64) + eps * d).sum() - f(x.astype(np.float64) - eps * d).sum()) / (2 * eps)
    assert abs(num - (dx.astype(np.float64) * d).sum()) < 1e-3 * max(1.0, abs(num))
    xh = ((xg - m) / np.sqrt(v + 1e-5)).reshape(B, HW, C)
    assert np.allclose(dg, (dy * xh).sum(axis=(0, 1)), atol=1e-4) and np.allclose(db, dy.sum(axis=(0, 1)), atol=1e-5)
    # layer norm and pixel norm
    xr = x.reshape(-1, C)
    yl, ml, rl = orc.layernorm_forward(xr, gam, bet, 1e-5)
    refl = (xr - xr.mean(1, keepdims=True)) / np.sqrt(xr.var(1, keepdims=True) + 1e-5) * gam + bet
    assert np.max(np.abs(yl - refl)) < 1e-5
    yp = orc.pixel_norm_forward(xr, 1e-4)
    assert np.max(np.abs(yp - xr / np.sqrt((xr.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-4))) < 1e-5


def test_weight_norm_and_adam_oracles_against_numpy(orc):
    rng = np.random.default_rng(4)
    W = rng.standard_normal((30, 7)).astype(np.float32)
    Wn = orc.weight_normalize(W, 1e-4)
    assert np.allclose(Wn, W / np.sqrt((W.astype(np.float64) ** 2).sum(0) + 1e-4), atol=1e-6)
    M = rng.standard_normal((30, 7)).astype(np.float32)
    gW, gg = orc.weight_normalize_backward(M, Wn, 1.7)
    dot = (Wn.astype(np.float64) * M).sum(0)
    assert np.allclose(gW, 1.7 * (M - dot * Wn), atol=1e-5) and abs(gg - dot.sum()) < 1e-4
    p = rng.standard_normal(100).astype(np.float32); g = rng.standard_normal(100).astype(np.float32)
    m0 = np.zeros(100, np.float32); v0 = np.zeros(100, np.float32)
    p1, m1, v1, s1 = orc.adam_ema_step(p, m0, v0, p, g, 1e-2, 0.9, 0.999, 1e-8, 0.1, 0.001, 0.99, 1.0)
    mm = 0.1 * g; vv = 0.001 * g * g
    pp = p - 1e-2 * (mm / 0.1) / (np.sqrt(vv / 0.001) + 1e-8)
    assert np.allclose(p1, pp, atol=1e-6) and np.allclose(s1, 0.99 * p + 0.01 * pp, atol=1e-6)
    a, b = orc.mp_cat(p.reshape(10, 10), g.reshape(10, 10), 0.5)[:, :10], None
    assert np.allclose(a, p.reshape(10, 10), atol=1e-6)  # t=0.5 with equal widths: unit weights


# ---- the launchers either side of the fused layer kernels (im2col/col2im, resampling, attention glue,
# ---- FiLM, bias and loss helpers): the oracle against golden outputs of the reference's kernels
import plain_cases as pc  # noqa: E402

GOLDEN_PLAIN = Path(__file__).resolve().parent / "golden" / "reference_plain_launchers.npz"


@pytest.fixture(scope="module")
def golden_plain():
    if not GOLDEN_PLAIN.exists():
        pytest.skip("golden file not generated yet")
    return np.load(GOLDEN_PLAIN)


@pytest.mark.parametrize("name,fn,args,tol", pc.PLAIN_CASES, ids=[c[0] for c in pc.PLAIN_CASES])
def test_plain_launcher_oracle_matches_reference_kernel_outputs(orc, golden_plain, name, fn, args, tol):
    arrays, _ = pc.materialise(name, args)
    flat = np.concatenate([np.ravel(v).astype(np.float64) for v in arrays.values()])
    assert np.allclose(golden_plain[f"{name}/__input_sum"], [flat.sum(), np.abs(flat).sum()], rtol=1e-12), \
        "seeded inputs differ from the ones the golden file was generated with"
    got = pc.run_oracle(orc, name, fn, args)
    pc.compare(got, {k: golden_plain[f"{name}/{k}"] for k in got}, tol, "oracle/" + name)
