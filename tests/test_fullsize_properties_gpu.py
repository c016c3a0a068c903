"""GPU: the baseline's FULL sizes, checked through size-independent properties (the CPU oracle
would take minutes at these sizes): normalisation invariants, linearity of the backward pass,
concat/split round trips, idempotence of the weight normalisation, sharded == unsharded."""
import importlib
import math

import pytest

pytestmark = pytest.mark.gpu


def _ops():
    return importlib.import_module("cuda-c-diffusion_b200.ops")


def test_groupnorm_cfg0_and_cfg2_invariants(lib):
    import torch
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(0)
    for (B, HW, C, G, act) in ((128, 784, 64, 32, None), (256, 1024, 256, 32, "silu")):
        x = torch.randn(B, HW, C, device="cuda", generator=g) * 1.7 + 0.3
        ones, zeros = torch.ones(C, device="cuda"), torch.zeros(C, device="cuda")
        # (1) with gamma=1, beta=0 and no activation every (sample, group) has mean 0 and variance 1
        y, mu, rstd = ops.groupnorm_forward(x, ones, zeros, G, 1e-5)
        yg = y.view(B, HW, G, C // G)
        assert float(yg.mean(dim=(1, 3)).abs().max()) < 2e-5
        assert float((yg.var(dim=(1, 3), unbiased=False) - 1).abs().max()) < 1e-4
        xg = x.view(B, HW, G, C // G)
        assert torch.allclose(mu.view(B, G), xg.mean(dim=(1, 3)), atol=1e-5)
        assert torch.allclose(rstd.view(B, G), (xg.var(dim=(1, 3), unbiased=False) + 1e-5).rsqrt(), rtol=1e-5)
        # (2) fused activation == activation applied to the plain output
        gam = 1 + 0.1 * torch.randn(C, device="cuda", generator=g); bet = 0.1 * torch.randn(C, device="cuda", generator=g)
        h, mu, rstd = ops.groupnorm_forward(x, gam, bet, G, 1e-5)
        if act:
            yf, mu2, rstd2 = ops.groupnorm_forward(x, gam, bet, G, 1e-5, act=act)
            assert torch.allclose(yf, ops.activation_forward(h, act), rtol=1e-5, atol=1e-6)
            assert torch.equal(mu, mu2) and torch.equal(rstd, rstd2)
        # (3) backward is linear in dy, dx sums to zero over each group when gamma is constant,
        #     and dbeta is the plain column sum of dy
        dy = torch.randn(B, HW, C, device="cuda", generator=g)
        dx1, dg1, db1 = ops.groupnorm_backward(dy, x, gam, bet, mu, rstd, G)
        dx2, dg2, db2 = ops.groupnorm_backward(2.5 * dy, x, gam, bet, mu, rstd, G)
        assert torch.allclose(dx2, 2.5 * dx1, rtol=1e-4, atol=1e-6)
        assert torch.allclose(dg2, 2.5 * dg1, rtol=1e-4, atol=1e-3) and torch.allclose(db2, 2.5 * db1, rtol=1e-4, atol=1e-3)
        assert torch.allclose(db1, dy.sum(dim=(0, 1)), rtol=1e-4, atol=2e-2)
        dxc, _, _ = ops.groupnorm_backward(dy, x, ones, zeros, mu, rstd, G)
        assert float(dxc.view(B, HW, G, C // G).sum(dim=(1, 3)).abs().max()) < 5e-2 * float(rstd.max())
        # (4) two runs are bit-identical (deterministic reductions)
        dx3, dg3, db3 = ops.groupnorm_backward(dy, x, gam, bet, mu, rstd, G)
        assert torch.equal(dx1, dx3) and torch.equal(dg1, dg3) and torch.equal(db1, db3)
        del x, y, h, dy, dx1, dx2, dx3, dxc
        torch.cuda.empty_cache()


def test_layernorm_cfg2_invariants(lib):
    import torch
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(1)
    rows, C = 262144, 256
    x = torch.randn(rows, C, device="cuda", generator=g) * 3 - 1
    y, mu, rstd = ops.layernorm_forward(x, torch.ones(C, device="cuda"), torch.zeros(C, device="cuda"), 1e-5)
    assert float(y.mean(dim=1).abs().max()) < 1e-5 and float((y.var(dim=1, unbiased=False) - 1).abs().max()) < 1e-4
    assert torch.allclose(mu, x.mean(dim=1), atol=1e-5)
    gam = 1 + 0.1 * torch.randn(C, device="cuda", generator=g)
    dy = torch.randn(rows, C, device="cuda", generator=g)
    dx, dg, db = ops.layernorm_backward(dy, x, gam, mu, rstd)
    assert torch.allclose(db, dy.sum(dim=0), rtol=1e-4, atol=5e-2)
    assert torch.allclose(dg, (dy * y).sum(dim=0), rtol=1e-4, atol=5e-2)
    assert float((dx * 1.0).sum(dim=1).abs().max()) < 1e-3   # rows of dx are orthogonal to the constant vector
    assert float((dx * y).sum(dim=1).abs().max()) < 2e-3     # ... and to the normalised row


def test_edm_op_set_cfg1_properties(lib):
    import torch
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(2)
    shape = (256, 28, 28, 128)
    a = torch.randn(shape, device="cuda", generator=g); b = torch.randn(shape, device="cuda", generator=g)
    # mp_sum preserves magnitude for independent unit-variance inputs; weights follow the closed form
    t = 0.3
    s = ops.mp_sum(a, b, t)
    d = math.sqrt((1 - t) ** 2 + t ** 2)
    assert torch.allclose(s, ((1 - t) / d) * a + (t / d) * b, rtol=1e-5, atol=1e-6)
    assert abs(float(s.var()) - 1.0) < 5e-3
    ga, gb = ops.mp_sum_backward(s, t)
    assert torch.allclose(ga, ((1 - t) / d) * s, rtol=1e-6, atol=0) and torch.allclose(gb, (t / d) * s, rtol=1e-6, atol=0)
    # mp_cat of two 64-channel tensors with t=0.5 has unit weights: split(cat) is the identity
    a64, b64 = a[..., :64].contiguous(), b[..., :64].contiguous()
    c = ops.mp_cat(a64, b64, 0.5)
    assert torch.equal(c[..., :64], a64) and torch.equal(c[..., 64:], b64)
    ra, rb = ops.mp_cat_backward(c, 0.5, 64, 64)
    assert torch.equal(ra, a64) and torch.equal(rb, b64)
    # MP-SiLU: odd part and scale; backward linear in the upstream gradient
    y = ops.activation_forward(a, "mp_silu")
    assert torch.allclose(y, ops.activation_forward(a, "silu") / 0.596, rtol=1e-6, atol=1e-7)
    g1 = ops.activation_backward(b, a, "mp_silu"); g2 = ops.activation_backward(3 * b, a, "mp_silu")
    assert torch.allclose(g2, 3 * g1, rtol=1e-6, atol=1e-7)
    # pixel norm: unit mean square per pixel, idempotent up to eps, dx orthogonal to x
    p = ops.pixel_norm_forward(a, 1e-4)
    assert float((p.pow(2).mean(dim=-1) - 1).abs().max()) < 2e-4
    dxp = ops.pixel_norm_backward(b, a, 1e-4)
    assert float((dxp * a).sum(dim=-1).abs().max()) < 2e-2
    # forced weight norm of the [3*3*128, 128] conv weight: unit columns, idempotent
    W = torch.randn(1152, 128, device="cuda", generator=g)
    ops.weight_normalize_(W, 1e-4)
    assert float((W.pow(2).sum(dim=0) - 1).abs().max()) < 1e-4
    W2 = W.clone()
    ops.weight_normalize_(W2, 1e-4)
    assert torch.allclose(W, W2, rtol=0, atol=1e-4)


def test_optimizer_cfg4_sharded_ranges_equal_unsharded(lib):
    """64M-parameter fused Adam+EMA: updating the 8 parameter ranges one by one (what 8 ranks do)
    gives bit-identical results to one flat launch, and the update moves against the gradient."""
    import torch
    ops = _ops()
    sh = importlib.import_module("cuda-c-diffusion_b200.sharding")
    n = 64 * 2 ** 20
    g = torch.Generator(device="cuda").manual_seed(3)
    p = 0.02 * torch.randn(n, device="cuda", generator=g); grad = 1e-3 * torch.randn(n, device="cuda", generator=g)
    hp = dict(lr=1e-4, b1=0.9, b2=0.999, eps=1e-8, bc1=0.1, bc2=0.001, decay=0.999)
    pa, ma, va, sa = p.clone(), torch.zeros_like(p), torch.zeros_like(p), p.clone()
    ops.adam_ema_step_(pa, ma, va, sa, grad, **hp)
    pb, mb, vb, sb = p.clone(), torch.zeros_like(p), torch.zeros_like(p), p.clone()
    for r in range(8):
        lo, hi = sh.param_range(n, r, 8)
        ops.adam_ema_step_(pb[lo:hi], mb[lo:hi], vb[lo:hi], sb[lo:hi], grad[lo:hi], **hp)
    assert torch.equal(pa, pb) and torch.equal(ma, mb) and torch.equal(va, vb) and torch.equal(sa, sb)
    step = pa - p
    assert float((step * grad).sum()) < 0 and float(step.abs().max()) <= 1e-3  # |step| ~ lr * m_hat / sqrt(v_hat)
    assert torch.allclose(sa, 0.999 * p + (1 - 0.999) * pa, rtol=1e-6, atol=1e-9)
