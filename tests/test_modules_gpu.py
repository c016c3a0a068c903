"""GPU: the host-side Module mirror driven the way the reference's tests/gradcheck.c drives its
modules (central differences of L = <forward(in), g>, EPS 1e-3, ATOL 1e-2, rtol 2e-2, batch 2),
extended to the fused modules the reference does not have, and the optimizer/EMA call sequences."""
import importlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

EPS, ATOL, RTOL, K = 1e-3, 1e-2, 2e-2, 20


def _mods():
    return importlib.import_module("reference_module_mirror")


def _check_module(m, batch, seed):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_in, n_out = batch * m.in_dim, batch * m.out_dim
    x = torch.randn(n_in, device="cuda", generator=g)
    cot = torch.randn(n_out, device="cuda", generator=g)
    out = torch.empty(n_out, device="cuda"); gin = torch.empty(n_in, device="cuda")
    pl = _mods().ParamList()
    m.parameters(pl)
    for it in pl:  # move parameters off their init values so that every gradient is exercised
        if it.size > 1:
            it.param.add_(0.3 * torch.randn(it.param.shape, device="cuda", generator=g))
    m.forward(x, out, batch)  # warm-up: projects in-place-normalised weights onto the sphere
    snaps = [it.param.clone() for it in pl]
    m.forward(x, out, batch)
    m.backward(x, out, cot, gin, batch)
    ana_in = gin.clone()
    ana_p = [it.grad.clone() for it in pl]

    def loss():
        m.forward(x, out, batch)
        return float((out.double() * cot.double()).sum())

    def restore():
        for it, s in zip(pl, snaps):
            it.param.copy_(s)

    rng = np.random.default_rng(seed)
    worst = 0.0
    for j in rng.choice(n_in, size=min(K, n_in), replace=False):
        save = float(x[j])
        restore(); x[j] = save + EPS; lp = loss()
        restore(); x[j] = save - EPS; lm = loss()
        x[j] = save
        num, ana = (lp - lm) / (2 * EPS), float(ana_in[j])
        worst = max(worst, abs(num - ana) / (ATOL + RTOL * (abs(num) + abs(ana))))
    for k, it in enumerate(pl):
        flat = it.param.view(-1)
        for j in rng.choice(it.size, size=min(K, it.size), replace=False):
            base = float(snaps[k].view(-1)[j])
            restore(); flat[j] = base + EPS; lp = loss()
            restore(); flat[j] = base - EPS; lm = loss()
            num, ana = (lp - lm) / (2 * EPS), float(ana_p[k].view(-1)[j])
            worst = max(worst, abs(num - ana) / (ATOL + RTOL * (abs(num) + abs(ana))))
    restore()
    return worst


@pytest.mark.parametrize("name", ["act_silu", "act_mp_silu", "act_gelu", "act_tanh", "layernorm", "groupnorm",
                                  "groupnorm_silu", "groupnorm_mp_silu", "pixel_norm", "mp_linear", "layernorm_256",
                                  "groupnorm_64x14x14"])
def test_finite_difference_gradients(lib, name):
    M = _mods()
    make = {
        "act_silu": lambda: M.activation_create(8, "silu"),
        "act_mp_silu": lambda: M.activation_create(8, "mp_silu"),
        "act_gelu": lambda: M.activation_create(8, "gelu"),
        "act_tanh": lambda: M.activation_create(8, "tanh"),
        "layernorm": lambda: M.layernorm_create(16, 2),
        "layernorm_256": lambda: M.layernorm_create(256, 2),
        "groupnorm": lambda: M.spatial_groupnorm_create(8, 4, 6, 6, 2),
        "groupnorm_silu": lambda: M.spatial_groupnorm_create(8, 4, 6, 6, 2, act="silu"),
        "groupnorm_mp_silu": lambda: M.spatial_groupnorm_create(16, 4, 5, 5, 2, act="mp_silu"),
        "groupnorm_64x14x14": lambda: M.spatial_groupnorm_create(64, 32, 14, 14, 2, act="silu"),
        "pixel_norm": lambda: M.PixelNorm(8, pixels_per_sample=4),
        "mp_linear": lambda: M.mp_linear_create(None, 12, 8, 1.0),
    }[name]
    worst = _check_module(make(), batch=2, seed=1234)
    assert worst <= 1.0, f"{name}: worst violation ratio {worst:.2f}"


def test_embeddings_have_no_backward_and_leave_grad_in_untouched(lib):
    import torch
    M = _mods()
    for m in (M.sinusoidal_create(16, 1e4), M.mp_fourier_create(None, 16, 1.0)):
        x = torch.rand(4, device="cuda") * 10
        out = torch.empty(4 * m.out_dim, device="cuda")
        gin = torch.full((4,), 7.0, device="cuda")
        m.forward(x, out, 4)
        m.backward(x, out, torch.ones_like(out), gin, 4)
        assert torch.all(gin == 7.0) and torch.isfinite(out).all()
    with pytest.raises(ValueError):
        M.sinusoidal_create(7, 1e4)


def test_fused_multi_tensor_update_equals_reference_call_sequence(lib):
    """optimizer_step (one launch per tensor) followed by ema_update == one fused multi-tensor launch."""
    import torch
    M = _mods()
    g = torch.Generator(device="cuda").manual_seed(5)
    sizes = [4096, 1, 300, 1, 73728]

    def build():
        pl = M.ParamList()
        gg = torch.Generator(device="cuda").manual_seed(5)
        for n in sizes:
            pl.add(0.02 * torch.randn(n, device="cuda", generator=gg), torch.zeros(n, device="cuda"), n)
        return pl

    pa, pb = build(), build()
    oa, ob = M.optimizer_adam(pa, 1e-3, 0.9, 0.999, 1e-8), M.optimizer_adam(pb, 1e-3, 0.9, 0.999, 1e-8)
    ea, eb = M.ema_create(pa, 0.999), M.ema_create(pb, 0.999)
    for _ in range(3):
        for a, b in zip(pa, pb):
            a.grad.copy_(1e-3 * torch.randn(a.size, device="cuda", generator=g)); b.grad.copy_(a.grad)
        oa.step(pa); ea.update(pa)
        ob.step_fused(pb, eb)
    assert oa.timestep() == ob.timestep() == 3
    for a, b, sa, sb in zip(pa, pb, ea.shadow, eb.shadow):
        assert torch.allclose(a.param, b.param, rtol=1e-6, atol=1e-8)
        assert torch.allclose(sa, sb, rtol=1e-6, atol=1e-8)
    ea.swap(pa)
    assert torch.allclose(pa[0].param, eb.shadow[0], rtol=1e-6, atol=1e-8)  # swap moved the shadow into the params
    assert abs(M.lr_inv_sqrt(1e-2, 5, 10, 100) - 5e-3) < 1e-12 and abs(M.lr_inv_sqrt(1e-2, 400, 10, 100) - 5e-3) < 1e-12
