"""GPU parity of the remaining launchers of the reference C ABI (the ones either
side of the fused layer kernels in a training step) against the CPU oracle."""
import ctypes

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu


_keep = []


def _t(a):
    """Host array -> device tensor that stays alive until the end of the test (a
    temporary would be freed, and its memory reused, before the kernel runs)."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    _keep.append(t)
    return t


@pytest.fixture(autouse=True)
def _release_device_tensors():
    yield
    _keep.clear()


def _st():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _n(t):
    return t.cpu().numpy()


F = ctypes.c_float
rng = np.random.default_rng(1234)
f = lambda *s: rng.standard_normal(s, dtype=np.float32)


@pytest.mark.parametrize("C", [4, 3, 16])
@pytest.mark.parametrize("K,stride,pad", [(3, 1, 1), (1, 1, 0), (3, 2, 1), (2, 1, 0), (5, 1, 2)])
def test_im2col_col2im(lib, orc, C, K, stride, pad):
    import torch
    B, H, W = 2, 6, 5
    Ho, Wo = (H + 2 * pad - K) // stride + 1, (W + 2 * pad - K) // stride + 1
    im = f(B, H, W, C)
    col = np.empty((B * Ho * Wo, K * K * C), np.float32)
    orc.raw("im2col", col, im, B, H, W, C, K, stride, pad, Ho, Wo)
    tim = _t(im); tcol = torch.empty(B * Ho * Wo, K * K * C, device="cuda")
    lib.launch_im2col(_p(tcol), _p(tim), B, H, W, C, K, stride, pad, Ho, Wo, _st())
    assert np.array_equal(_n(tcol), col)
    gcol = f(B * Ho * Wo, K * K * C)
    gim = np.zeros((B, H, W, C), np.float32)
    orc.raw("col2im", gim, gcol, B, H, W, C, K, stride, pad, Ho, Wo)
    tg = torch.zeros(B, H, W, C, device="cuda")
    lib.launch_col2im(_p(tg), _p(_t(gcol)), B, H, W, C, K, stride, pad, Ho, Wo, _st())
    assert cases.rel_err(_n(tg), gim) <= 1e-6
    # the overwriting variant gives the same result on a buffer full of garbage
    ta = torch.full((B, H, W, C), 123.0, device="cuda")
    lib.launch_col2im_assign(_p(ta), _p(_t(gcol)), B, H, W, C, K, stride, pad, Ho, Wo, _st())
    assert torch.equal(ta, tg)


@pytest.mark.parametrize("C", [8, 5])
def test_resampling(lib, orc, C):
    import torch
    B, H, W = 2, 6, 4
    x = f(B, H, W, C)
    ref = np.empty((B, H // 2, W // 2, C), np.float32)
    orc.raw("avg_pool_2x", ref, x, B, H, W, C)
    out = torch.empty(B, H // 2, W // 2, C, device="cuda")
    lib.launch_avg_pool_2x(_p(out), _p(_t(x)), B, H, W, C, _st())
    assert cases.rel_err(_n(out), ref) <= 1e-6
    g = f(B, H // 2, W // 2, C)
    refg = np.zeros((B, H, W, C), np.float32)
    orc.raw("avg_pool_2x_backward", refg, g, B, H, W, C)
    outg = torch.zeros(B, H, W, C, device="cuda")
    lib.launch_avg_pool_2x_backward(_p(outg), _p(_t(g)), B, H, W, C, _st())
    assert np.array_equal(_n(outg), refg)
    refu = np.empty((B, 2 * H, 2 * W, C), np.float32)
    orc.raw("nearest_upsample_2x", refu, x, B, H, W, C)
    outu = torch.empty(B, 2 * H, 2 * W, C, device="cuda")
    lib.launch_nearest_upsample_2x(_p(outu), _p(_t(x)), B, H, W, C, _st())
    assert np.array_equal(_n(outu), refu)
    gu = f(B, 2 * H, 2 * W, C)
    refgu = np.empty((B, H, W, C), np.float32)
    orc.raw("nearest_upsample_2x_backward", refgu, gu, B, H, W, C)
    outgu = torch.empty(B, H, W, C, device="cuda")
    lib.launch_nearest_upsample_2x_backward(_p(outgu), _p(_t(gu)), B, H, W, C, _st())
    assert cases.rel_err(_n(outgu), refgu) <= 1e-6


def test_attention_glue(lib, orc):
    import torch
    N, S = 37, 49
    x = f(N, S) * 3
    ref = np.empty_like(x)
    orc.raw("attn_softmax", ref, x, N, S)
    tx = _t(x)
    out = torch.empty_like(tx)
    lib.launch_attn_softmax(_p(out), _p(tx), N, S, _st())
    assert cases.rel_err(_n(out), ref) <= 1e-5
    lib.launch_attn_softmax(_p(tx), _p(tx), N, S, _st())  # in place, as attention.c calls it
    assert cases.rel_err(_n(tx), ref) <= 1e-5
    g = f(N, S)
    refg = np.empty_like(x)
    orc.raw("attn_softmax_backward", refg, g, ref, N, S)
    outg = torch.empty_like(tx)
    lib.launch_attn_softmax_backward(_p(outg), _p(_t(g)), _p(_t(ref)), N, S, _st())
    assert cases.rel_err(_n(outg), refg) <= 1e-4
    for d3 in (8, 3):
        B, d1, d2 = 2, 5, 4
        y = f(B, d1, d2, d3)
        refp = np.empty((B, d2, d1, d3), np.float32)
        orc.raw("permute_0213", refp, y, B, d1, d2, d3)
        outp = torch.empty(B, d2, d1, d3, device="cuda")
        lib.launch_permute_0213(_p(outp), _p(_t(y)), B, d1, d2, d3, _st())
        assert np.array_equal(_n(outp), refp)


@pytest.mark.parametrize("C", [64, 6])
def test_film_and_spatial_bias(lib, orc, C):
    import torch
    B, H, W = 3, 7, 7
    x, cond, g = f(B, H, W, C), f(B, C), f(B, H, W, C)
    ref = np.empty_like(x)
    orc.raw("spatial_modulate", ref, x, cond, B, H, W, C)
    out = torch.empty(B, H, W, C, device="cuda")
    lib.launch_spatial_modulate(_p(out), _p(_t(x)), _p(_t(cond)), B, H, W, C, _st())
    assert cases.rel_err(_n(out), ref) <= 1e-6
    rgi, rgc = np.empty_like(x), np.empty_like(cond)
    orc.raw("spatial_modulate_backward", rgi, rgc, g, x, cond, B, H, W, C)
    gi, gc = torch.empty(B, H, W, C, device="cuda"), torch.empty(B, C, device="cuda")
    lib.launch_spatial_modulate_backward(_p(gi), _p(gc), _p(_t(g)), _p(_t(x)), _p(_t(cond)), B, H, W, C, _st())
    assert cases.rel_err(_n(gi), rgi) <= 1e-6
    assert cases.rel_err(_n(gc), rgc) <= 1e-4
    xa = x.copy()
    orc.raw("spatial_add", xa, cond, B, H, W, C)
    tx = _t(x)
    lib.launch_spatial_add(_p(tx), _p(_t(cond)), B, H, W, C, _st())
    assert cases.rel_err(_n(tx), xa) <= 1e-6
    rs = np.empty((B, C), np.float32)
    orc.raw("spatial_reduce_sum", rs, x, B, H * W, C)
    ts = torch.empty(B, C, device="cuda")
    lib.launch_spatial_reduce_sum(_p(ts), _p(_t(x)), B, H * W, C, _st())
    assert cases.rel_err(_n(ts), rs) <= 1e-5


def test_dense_head_helpers(lib, orc):
    import torch
    M, N = 9, 12
    Y, b, g = f(M, N), f(N), f(M, N)
    ya = Y.copy()
    orc.raw("add_bias", ya, b, M, N)
    ty = _t(Y)
    lib.launch_add_bias(_p(ty), _p(_t(b)), M, N, _st())
    assert cases.rel_err(_n(ty), ya) <= 1e-6
    rb = np.empty(N, np.float32)
    orc.raw("bias_grad", rb, g, M, N)
    tb = torch.empty(N, device="cuda")
    lib.launch_bias_grad(_p(tb), _p(_t(g)), M, N, _st())
    assert cases.rel_err(_n(tb), rb) <= 1e-5
    # MSE head
    B, dim = 5, 784
    pred, tgt = f(B, dim), f(B, dim)
    rg, rl = np.empty_like(pred), np.empty(B, np.float32)
    orc.raw("mse_fwd_bwd", rg, rl, pred, tgt, B, dim)
    tg, tl = torch.empty(B, dim, device="cuda"), torch.empty(B, device="cuda")
    lib.launch_mse_fwd_bwd(_p(tg), _p(tl), _p(_t(pred)), _p(_t(tgt)), B, dim, _st())
    assert cases.rel_err(_n(tg), rg) <= 1e-6 and cases.rel_err(_n(tl), rl) <= 1e-5
    # softmax cross-entropy head
    Bc, C = 6, 10
    z = f(Bc, C) * 2
    tgts = rng.integers(0, C, Bc).astype(np.int32)
    rgz, rlz = np.empty_like(z), np.empty(Bc, np.float32)
    orc.raw("softmax_xent", rgz, rlz, z, tgts, Bc, C)
    tgz, tlz = torch.empty(Bc, C, device="cuda"), torch.empty(Bc, device="cuda")
    lib.launch_softmax_xent(_p(tgz), _p(tlz), _p(_t(z)), _p(_t(tgts)), Bc, C, _st())
    assert cases.rel_err(_n(tgz), rgz) <= 1e-5 and cases.rel_err(_n(tlz), rlz) <= 1e-5
    # clamp, sgd, modulate
    x = f(1001) * 3
    xc = x.copy()
    orc.raw("clamp", xc, -1.0, 2.0, orc.L(x.size))
    tx = _t(x)
    lib.launch_clamp(_p(tx), F(-1.0), F(2.0), x.size, _st())
    assert np.array_equal(_n(tx), xc)
    p0, g0 = f(777), f(777)
    pr = p0.copy()
    orc.raw("sgd_step", pr, g0, 0.1, orc.L(777))
    tp = _t(p0)
    lib.launch_sgd_step(_p(tp), _p(_t(g0)), F(0.1), 777, _st())
    assert cases.rel_err(_n(tp), pr) <= 1e-6
    h1, c, gh2 = f(500), f(500), f(500)
    r2 = np.empty_like(h1)
    orc.raw("modulate", r2, h1, c, orc.L(500))
    t2 = torch.empty(500, device="cuda")
    lib.launch_modulate(_p(t2), _p(_t(h1)), _p(_t(c)), 500, _st())
    assert cases.rel_err(_n(t2), r2) <= 1e-6
    rgh, rgc = np.empty_like(h1), np.empty_like(h1)
    orc.raw("modulate_backward", rgh, rgc, gh2, h1, c, orc.L(500))
    tgh, tgc = torch.empty(500, device="cuda"), torch.empty(500, device="cuda")
    lib.launch_modulate_backward(_p(tgh), _p(tgc), _p(_t(gh2)), _p(_t(h1)), _p(_t(c)), 500, _st())
    assert cases.rel_err(_n(tgh), rgh) <= 1e-6 and cases.rel_err(_n(tgc), rgc) <= 1e-6


def test_learned_embedding_table(lib, orc):
    import torch
    T, C, B = 7, 12, 9
    table, go = f(T, C), f(B, C)
    idx = np.array([0, 3, 3, 6, 9, -2, 1, 1, 1], np.float32)  # out-of-range indices are clamped
    ref = np.empty((B, C), np.float32)
    orc.raw("embed_gather", ref, table, idx, B, C, T)
    out = torch.empty(B, C, device="cuda")
    lib.launch_embed_gather(_p(out), _p(_t(table)), _p(_t(idx)), B, C, T, _st())
    assert np.array_equal(_n(out), ref)
    rg = np.zeros((T, C), np.float32)
    orc.raw("embed_scatter", rg, go, idx, B, C, T)
    tg = torch.zeros(T, C, device="cuda")
    lib.launch_embed_scatter(_p(tg), _p(_t(go)), _p(_t(idx)), B, C, T, _st())
    assert cases.rel_err(_n(tg), rg) <= 1e-5


def test_channel_cat_split_plain(lib, orc):
    import torch
    for Ca, Cb in ((64, 32), (5, 3)):
        rows = 41
        a, b, g = f(rows, Ca), f(rows, Cb), f(rows, Ca + Cb)
        out = torch.empty(rows, Ca + Cb, device="cuda")
        lib.launch_channel_cat(_p(out), _p(_t(a)), _p(_t(b)), rows, Ca, Cb, _st())
        assert np.array_equal(_n(out), orc.channel_cat(a, b))
        ga, gb = torch.empty(rows, Ca, device="cuda"), torch.empty(rows, Cb, device="cuda")
        lib.launch_channel_split(_p(ga), _p(gb), _p(_t(g)), rows, Ca, Cb, _st())
        ra, rb = orc.channel_split(g, Ca, Cb)
        assert np.array_equal(_n(ga), ra) and np.array_equal(_n(gb), rb)


@pytest.mark.parametrize("B,H,W,C", [(3, 7, 7, 24), (2, 32, 32, 32), (5, 9, 4, 6), (64, 14, 14, 128)])
@pytest.mark.parametrize("act", [5, 3, 0])
def test_fused_residual_block_passes_match_their_compositions(lib, B, H, W, C, act):
    """launch_film_act_forward / _backward and launch_activation_backward_axpy against the sequences of
    reference launchers they replace (cond_conv_residual.c:31-33, :49-54, :54+:61)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + C)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    h1, cond, gout, skip = rn(B, H, W, C), 0.3 * rn(B, C), rn(B, H, W, C), rn(B, H, W, C)
    n = h1.numel()
    # forward
    h2, want = torch.empty_like(h1), torch.empty_like(h1)
    lib.launch_spatial_modulate(_p(h2), _p(h1), _p(cond), B, H, W, C, _st())
    lib.launch_activation_forward(_p(want), _p(h2), n, act, _st())
    got = torch.empty_like(h1)
    lib.launch_film_act_forward(_p(got), _p(h1), _p(cond), B, H, W, C, act, _st())
    assert torch.equal(got, want)
    # backward
    gh2, gh1_want, gc_want = torch.empty_like(h1), torch.empty_like(h1), torch.empty(B, C, device="cuda")
    lib.launch_activation_backward(_p(gh2), _p(gout), _p(h2), n, act, _st())
    lib.launch_spatial_modulate_backward(_p(gh1_want), _p(gc_want), _p(gh2), _p(h1), _p(cond), B, H, W, C, _st())
    gh1, gc = torch.empty_like(h1), torch.full((B, C), 7.0, device="cuda")
    lib.launch_film_act_backward(_p(gh1), _p(gc), _p(gout), _p(h1), _p(cond), B, H, W, C, act, _st())
    torch.cuda.synchronize()
    assert cases.rel_err(_n(gh1), _n(gh1_want)) <= 1e-6
    assert cases.rel_err(_n(gc), _n(gc_want)) <= 2e-5  # different summation order over H*W
    # activation backward + skip
    gx, want2 = torch.empty_like(h1), torch.empty_like(h1)
    lib.launch_activation_backward(_p(gx), _p(gout), _p(h1), n, act, _st())
    lib.launch_weighted_sum(_p(want2), _p(skip), _p(gx), F(0.8), F(1.0), n, _st())
    got2 = torch.empty_like(h1)
    lib.launch_activation_backward_axpy(_p(got2), _p(gout), _p(h1), _p(skip), F(0.8), n, act, _st())
    torch.cuda.synchronize()
    assert cases.rel_err(_n(got2), _n(want2)) <= 1e-6
