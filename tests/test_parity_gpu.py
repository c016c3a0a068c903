"""GPU parity: the CUDA library, called through its C ABI, against the CPU oracle
and against the reference's own kernels rebuilt for sm_100a (A/B), on the same
seeded inputs.  Tolerances are the stated fp32 ones: forward rel <= 1e-5,
backward rel <= 1e-4 (cases.TOL_FWD / TOL_BWD), relative to the largest
reference magnitude of the tensor."""
import ctypes
import math

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu

EXTRA = [
    ("pixel_norm_128", "pixel_norm", dict(rows=77, C=128, eps=1e-4)),
    ("pixel_norm_24", "pixel_norm", dict(rows=9, C=24, eps=1e-4)),
    ("layernorm_384", "layernorm", dict(rows=70, C=384)),
    ("layernorm_1024", "layernorm", dict(rows=19, C=1024)),
    ("layernorm_100", "layernorm", dict(rows=300, C=100)),
    ("groupnorm_g8", "groupnorm", dict(B=3, HW=256, C=64, G=8, act=None)),
    ("groupnorm_mp_silu", "groupnorm", dict(B=2, HW=196, C=128, G=32, act="mp_silu")),
    ("groupnorm_relu", "groupnorm", dict(B=1, HW=64, C=16, G=2, act="relu")),
    ("groupnorm_wide", "groupnorm", dict(B=2, HW=1024, C=256, G=32, act="silu")),
    ("groupnorm_cpg1", "groupnorm", dict(B=2, HW=100, C=32, G=32, act=None)),
    ("groupnorm_96", "groupnorm", dict(B=2, HW=64, C=96, G=32, act=None)),
    ("weight_norm_big", "weight_norm", dict(rows=1152, cols=128, eps=1e-4)),
    ("weight_norm_tall", "weight_norm", dict(rows=2500, cols=20, eps=1e-4)),
    ("weight_norm_tiny", "weight_norm", dict(rows=3, cols=4, eps=1e-4)),
    ("adam_ema_odd", "adam_ema", dict(n=4099, steps=2, decay=0.99)),
    ("mp_cat_wide", "mp_cat", dict(rows=513, Ca=128, Cb=64, t=0.7)),
]
ALL = cases.CASES + EXTRA


def _check(got, ref, name, skip=()):
    for k, r in ref.items():
        if k in skip or k == "y64":
            continue
        e = cases.rel_err(got[k], r)
        assert e <= cases.tolerance(k), f"{name}:{k} rel err {e:.3e} > {cases.tolerance(k):.0e}"


def _embedding_check(got, ref64, tmax, name):
    # sin/cos of an fp32 argument of magnitude A carries an absolute error of about
    # A * 2^-23 from rounding the argument alone; allow a few units of that.
    tol = 4.0 * max(tmax, 1.0) * 2.0 ** -23 + 2e-6
    err = float(np.max(np.abs(got.astype(np.float64) - ref64)))
    assert err <= tol, f"{name}: abs err {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("name,op,p", ALL, ids=[c[0] for c in ALL])
def test_matches_oracle(lib, orc, name, op, p):
    inp = cases.make_inputs(op, p, seed=cases.seed_of(name))
    ref = cases.oracle_run(orc, op, p, inp)
    got = cases.gpu_run(lib, op, p, inp, fused=True)
    if op == "mp_fourier":
        _embedding_check(got["y"], ref["y64"], 2 * math.pi * 4.0, name)
    elif op == "sinusoidal":
        _embedding_check(got["y"], ref["y64"], p["tmax"], name)
    else:
        _check(got, ref, name)


REF_CASES = [c for c in ALL if c[1] != "pixel_norm"]


@pytest.mark.parametrize("name,op,p", REF_CASES, ids=[c[0] for c in REF_CASES])
def test_matches_reference_kernels(lib, ref_lib, ref_lib_precise, name, op, p):
    """A/B against the reference's kernels.cu built for this GPU.  Embeddings use the
    build without --use_fast_math: the fast intrinsics are off by far more than
    the tolerance at these arguments."""
    inp = cases.make_inputs(op, p, seed=cases.seed_of(name))
    got = cases.gpu_run(lib, op, p, inp, fused=True)
    if op in ("mp_fourier", "sinusoidal"):
        ref = cases.gpu_run(ref_lib_precise, op, p, inp, fused=False)
        tmax = p.get("tmax", 2 * math.pi * 4.0)
        _embedding_check(got["y"], ref["y"].astype(np.float64), 2 * tmax, name)
        return
    ref = cases.gpu_run(ref_lib, op, p, inp, fused=False)
    _check(got, ref, name)


def test_oracle_agrees_with_reference_kernels(orc, ref_lib):
    """Pins the CPU restatement to the reference itself on every non-embedding case."""
    for name, op, p in cases.CASES:
        if op in ("mp_fourier", "sinusoidal"):
            continue
        inp = cases.make_inputs(op, p, seed=cases.seed_of(name))
        _check(cases.oracle_run(orc, op, p, inp), cases.gpu_run(ref_lib, op, p, inp, fused=False), "oracle/" + name)


# ----------------------------------------------------------------------------- edge cases
def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


def _st():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _pp(t, off=0):
    return ctypes.c_void_p(t.data_ptr() + 4 * off)


def test_empty_and_single_element(lib):
    import torch
    x = torch.ones(8, device="cuda")
    y = torch.zeros(8, device="cuda")
    lib.launch_activation_forward(_pp(y), _pp(x), 0, 3, _st())
    lib.launch_weighted_sum(_pp(y), _pp(x), _pp(x), ctypes.c_float(1), ctypes.c_float(1), 0, _st())
    lib.launch_groupnorm_forward(_pp(y), _pp(y), _pp(y), _pp(x), _pp(x), _pp(x), 0, 4, 4, 2, ctypes.c_float(1e-5), _st())
    torch.cuda.synchronize()
    assert float(y.abs().sum()) == 0.0
    lib.launch_activation_forward(_pp(y), _pp(x), 1, 1, _st())
    torch.cuda.synchronize()
    assert y[0].item() == 1.0 and float(y[1:].abs().sum()) == 0.0


def test_misaligned_pointers_take_the_scalar_path(lib, orc):
    import torch
    rng = np.random.default_rng(5)
    a = rng.standard_normal(1027, dtype=np.float32)
    b = rng.standard_normal(1027, dtype=np.float32)
    ta, tb = _t(a), _t(b)
    out = torch.zeros(1027, device="cuda")
    n = 1021
    lib.launch_weighted_sum(_pp(out, 3), _pp(ta, 1), _pp(tb, 2), ctypes.c_float(0.5), ctypes.c_float(2.0), n, _st())
    torch.cuda.synchronize()
    ref = orc.weighted_sum(a[1:1 + n], b[2:2 + n], 0.5, 2.0)
    got = out.cpu().numpy()
    assert cases.rel_err(got[3:3 + n], ref) <= 1e-6
    assert np.all(got[:3] == 0) and np.all(got[3 + n:] == 0)
    # misaligned groupnorm falls back to the generic kernels and still matches
    B, HW, C, G = 2, 64, 32, 4
    x = rng.standard_normal(B * HW * C + 1, dtype=np.float32)
    gam = rng.standard_normal(C, dtype=np.float32); bet = rng.standard_normal(C, dtype=np.float32)
    tx, tg, tbt = _t(x), _t(gam), _t(bet)
    y = torch.zeros(B * HW * C + 1, device="cuda"); mu = torch.zeros(B * G, device="cuda"); rs = torch.zeros(B * G, device="cuda")
    lib.launch_groupnorm_forward(_pp(y, 1), _pp(mu), _pp(rs), _pp(tx, 1), _pp(tg), _pp(tbt), B, HW, C, G,
                                 ctypes.c_float(1e-5), _st())
    torch.cuda.synchronize()
    ry, rmu, rrs = orc.groupnorm_forward(x[1:].reshape(B, HW, C), gam, bet, G, 1e-5)
    assert cases.rel_err(y.cpu().numpy()[1:], ry.ravel()) <= 1e-5


def test_aliased_operands_of_weighted_sum(lib, orc):
    """out==a (ema.c:32, unet.c:247) and a==b (edm.c:57) are legal in the reference."""
    import torch
    rng = np.random.default_rng(6)
    a = rng.standard_normal(5000, dtype=np.float32); b = rng.standard_normal(5000, dtype=np.float32)
    ta, tb = _t(a), _t(b)
    lib.launch_weighted_sum(_pp(ta), _pp(ta), _pp(tb), ctypes.c_float(0.999), ctypes.c_float(0.001), 5000, _st())
    torch.cuda.synchronize()
    assert cases.rel_err(ta.cpu().numpy(), orc.weighted_sum(a, b, 0.999, 0.001)) <= 1e-6
    tb2 = _t(b)
    lib.launch_weighted_sum(_pp(tb2), _pp(tb2), _pp(tb2), ctypes.c_float(0.25), ctypes.c_float(0.5), 5000, _st())
    torch.cuda.synchronize()
    assert cases.rel_err(tb2.cpu().numpy(), orc.weighted_sum(b, b, 0.25, 0.5)) <= 1e-6


def test_backward_overwrites_parameter_gradients_and_is_deterministic(lib):
    """Parameter gradients are overwritten (never accumulated) and two runs are bit-identical."""
    import torch
    name, op, p = "gn_det", "groupnorm", dict(B=6, HW=196, C=64, G=32, act="silu")
    inp = cases.make_inputs(op, p, seed=11)
    r1 = cases.gpu_run(lib, op, p, inp, fused=True)
    r2 = cases.gpu_run(lib, op, p, inp, fused=True)
    for k in r1:
        assert np.array_equal(r1[k], r2[k]), k
    name, op, p = "ln_det", "layernorm", dict(rows=1000, C=256)
    inp = cases.make_inputs(op, p, seed=12)
    r1 = cases.gpu_run(lib, op, p, inp, fused=True)
    r2 = cases.gpu_run(lib, op, p, inp, fused=True)
    for k in r1:
        assert np.array_equal(r1[k], r2[k]), k


def test_strip_and_generic_groupnorm_agree(lib, orc):
    """The generic kernels (any shape and alignment) on a shape the register strips normally take."""
    p = dict(B=4, HW=196, C=64, G=32, act="silu")
    inp = cases.make_inputs("groupnorm", p, seed=21)
    strips = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    lib.b200_tune_set(b"gn_force_generic", 1)
    try:
        gen = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    finally:
        lib.b200_tune_set(b"gn_force_generic", 0)
    ref = cases.oracle_run(orc, "groupnorm", p, inp)
    _check(strips, ref, "strips")
    _check(gen, ref, "generic")


STRIP_KEYS = (b"gn_fwd_strip_nt", b"gn_bwd_strip_nt", b"gn_fwd_strip_ct", b"gn_bwd_strip_ct", b"gn_bwd_strip_vpt")


@pytest.mark.parametrize("nt,fct,bct,bvpt", [(1024, 32, 16, 4), (512, 16, 8, 4), (1024, 8, 8, 4), (256, 8, 4, 4),
                                             (512, 16, 16, 8), (512, 8, 8, 8)])
def test_groupnorm_strip_geometries(lib, orc, nt, fct, bct, bvpt):
    """The register-resident strip kernels with forced CTA size and strip width (ragged HW:
    196 rows do not divide evenly over the row lanes)."""
    p = dict(B=5, HW=196, C=64, G=32, act="silu")
    inp = cases.make_inputs("groupnorm", p, seed=35)
    ref = cases.oracle_run(orc, "groupnorm", p, inp)
    for key, val in zip(STRIP_KEYS, (nt, nt, fct, bct, bvpt)):
        lib.b200_tune_set(key, val)
    try:
        n0 = lib.b200_launch_count()
        got = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
        assert lib.b200_launch_count() - n0 == 3, "expected the forward strip, backward strip and fold kernels"
    finally:
        for key in STRIP_KEYS:
            lib.b200_tune_set(key, 0)
        lib.b200_tune_set(b"gn_bwd_strip_vpt", 8)
    _check(got, ref, f"strip nt{nt}")


@pytest.mark.parametrize("shape", [dict(B=3, HW=4096, C=32, G=8), dict(B=2, HW=2500, C=48, G=6),
                                   dict(B=80, HW=4100, C=64, G=32)])
@pytest.mark.parametrize("act", ["silu", "mp_silu", None])
@pytest.mark.parametrize("bwd_vpt", [8, 4])
def test_groupnorm_chunked_strips_for_tall_samples(lib, orc, shape, act, bwd_vpt):
    """Samples too tall for the register-resident strips (64x64 images, ragged 50x50, and enough strips
    that every CTA loops over several): the chunked two-pass strip kernels are taken."""
    p = dict(shape, act=act)
    inp = cases.make_inputs("groupnorm", p, seed=41)
    ref = cases.oracle_run(orc, "groupnorm", p, inp)
    lib.b200_tune_set(b"gn_bwd_cstrip_vpt", bwd_vpt)
    try:
        n0 = lib.b200_launch_count()
        got = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
        assert lib.b200_launch_count() - n0 == 3, "expected chunked forward, chunked backward and the fold kernel"
        got2 = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    finally:
        lib.b200_tune_set(b"gn_bwd_cstrip_vpt", 8)
    _check(got, ref, "chunked strips")
    for k in got:
        assert np.array_equal(got[k], got2[k]), k


@pytest.mark.parametrize("bwd_pipeline", [0, 1])
def test_groupnorm_pipelined_strips(lib, orc, bwd_pipeline):
    """Many more strips than resident CTAs: the persistent kernels that prefetch the next strip with
    cp.async are taken (forward by default, backward on request) and loop several times."""
    p = dict(B=320, HW=1024, C=32, G=8, act="silu")
    lib.b200_tune_set(b"gn_bwd_pipeline", bwd_pipeline)  # 0 = plain strips
    inp = cases.make_inputs("groupnorm", p, seed=37)
    ref = cases.oracle_run(orc, "groupnorm", p, inp)
    try:
        got = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
        got2 = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    finally:
        for key in STRIP_KEYS:
            lib.b200_tune_set(key, 0)
        lib.b200_tune_set(b"gn_bwd_strip_vpt", 8)
        lib.b200_tune_set(b"gn_bwd_pipeline", 1)
    _check(got, ref, "pipelined")
    for k in got:
        assert np.array_equal(got[k], got2[k]), k


def test_multi_tensor_entry_points(pkg, lib, orc):
    import importlib
    import torch
    ops = importlib.import_module("cuda-c-diffusion_b200.ops")
    rng = np.random.default_rng(41)
    sizes = [1, 7, 4096, 1, 73728, 128, 1, 36864]
    P = [rng.standard_normal(n, dtype=np.float32) * 0.02 for n in sizes]
    Gd = [rng.standard_normal(n, dtype=np.float32) * 1e-3 for n in sizes]
    tp = [_t(x) for x in P]; tg = [_t(x) for x in Gd]
    tm = [torch.zeros_like(x) for x in tp]; tv = [torch.zeros_like(x) for x in tp]; ts = [x.clone() for x in tp]
    ts[1] = None  # a tensor without EMA shadow
    bc1, bc2 = cases._bias_corrections(1)
    ops.adam_ema_step_multi_(zip(tp, tg, tm, tv, ts), 1e-3, 0.9, 0.999, 1e-8, bc1, bc2, 0.999, 0.5)
    torch.cuda.synchronize()
    for i, n in enumerate(sizes):
        rp, rm, rv, rsh = orc.adam_ema_step(P[i], np.zeros(n, np.float32), np.zeros(n, np.float32), P[i], Gd[i], 1e-3,
                                            0.9, 0.999, 1e-8, bc1, bc2, 0.999, 0.5)
        assert cases.rel_err(tp[i].cpu().numpy(), rp) <= 1e-5, i
        assert cases.rel_err(tm[i].cpu().numpy(), rm) <= 1e-5, i
        assert cases.rel_err(tv[i].cpu().numpy(), rv) <= 1e-5, i
        if ts[i] is not None:
            assert cases.rel_err(ts[i].cpu().numpy(), rsh) <= 1e-5, i
    shapes = [(1152, 128), (64, 128), (576, 64), (9, 64), (30, 6)]
    Ws = [rng.standard_normal(s, dtype=np.float32) for s in shapes]
    tw = [_t(w) for w in Ws]
    ops.weight_normalize_multi_(tw, 1e-4)
    torch.cuda.synchronize()
    for w, t in zip(Ws, tw):
        assert cases.rel_err(t.cpu().numpy(), orc.weight_normalize(w, 1e-4)) <= 1e-5


def test_weight_normalize_backward_multi_and_batching_session(lib, capi):
    """One launch for several weights equals the per-weight launches; the record / batched session
    (what a training loop over the reference's unmodified modules uses) gives the same results."""
    import torch
    rng = np.random.default_rng(77)
    shapes = [(1152, 128), (64, 128), (576, 64), (128, 128), (9, 64), (30, 6)]
    W = [_t(rng.standard_normal(s, dtype=np.float32)) for s in shapes]
    for w, (i, o) in zip(W, shapes):
        lib.launch_weight_normalize(_pp(w), i, o, ctypes.c_float(1e-4), _st())
    G0 = [_t(rng.standard_normal(s, dtype=np.float32)) for s in shapes]
    gains = [_t(np.array([0.5 + 0.25 * k], np.float32)) for k in range(len(shapes))]

    def single():
        g = [x.clone() for x in G0]
        gg = [torch.zeros(1, device="cuda") for _ in shapes]
        for k, (i, o) in enumerate(shapes):
            lib.launch_weight_normalize_backward(_pp(g[k]), _pp(W[k]), _pp(gains[k]), _pp(gg[k]), i, o, _st())
        torch.cuda.synchronize()
        return g, gg

    ref_g, ref_gg = single()
    g = [x.clone() for x in G0]
    gg = [torch.zeros(1, device="cuda") for _ in shapes]
    arr = (capi.WeightGradDesc * len(shapes))()
    for k, (i, o) in enumerate(shapes):
        arr[k] = capi.WeightGradDesc(g[k].data_ptr(), W[k].data_ptr(), gains[k].data_ptr(), gg[k].data_ptr(), i, o)
    n0 = lib.b200_launch_count()
    lib.launch_weight_normalize_backward_multi(ctypes.cast(arr, ctypes.c_void_p), len(shapes), _st())
    torch.cuda.synchronize()
    assert lib.b200_launch_count() - n0 == 2  # one table launch + the one shape (30x6) outside the cluster kernel
    for k in range(len(shapes)):
        # (the table launch uses clusters of 8 for every matrix, so column dots fold in another order)
        assert cases.rel_err(g[k].cpu().numpy(), ref_g[k].cpu().numpy()) <= 2e-6, k
        assert abs(float(gg[k]) - float(ref_gg[k])) <= 1e-5 * max(1.0, abs(float(ref_gg[k]))), k

    # session: record one pass, then batched passes
    try:
        raw = [_t(rng.standard_normal(s, dtype=np.float32)) for s in shapes]
        expect = [x.clone() for x in raw]
        for w, (i, o) in zip(expect, shapes):
            lib.launch_weight_normalize(_pp(w), i, o, ctypes.c_float(1e-4), _st())
        lib.b200_wn_batch_mode(1)
        scratch = [x.clone() for x in raw]
        for w, (i, o) in zip(scratch, shapes):
            lib.launch_weight_normalize(_pp(w), i, o, ctypes.c_float(1e-4), _st())
        lib.b200_wn_batch_mode(2)
        for w, x in zip(scratch, raw):
            w.copy_(x)  # "the optimizer changed the weights"
        assert lib.b200_wn_forward_all(_st()) == len(shapes)
        n0 = lib.b200_launch_count()
        for w, (i, o) in zip(scratch, shapes):  # the modules' own calls are no-ops now
            lib.launch_weight_normalize(_pp(w), i, o, ctypes.c_float(1e-4), _st())
        g2 = [x.clone() for x in G0]
        gg2 = [torch.zeros(1, device="cuda") for _ in shapes]
        for k, (i, o) in enumerate(shapes):  # queued, not launched
            lib.launch_weight_normalize_backward(_pp(g2[k]), _pp(W[k]), _pp(gains[k]), _pp(gg2[k]), i, o, _st())
        assert lib.b200_launch_count() == n0
        assert lib.b200_wn_backward_flush(_st()) == len(shapes)
        assert lib.b200_wn_backward_flush(_st()) == 0
        torch.cuda.synchronize()
        for k in range(len(shapes)):
            assert cases.rel_err(scratch[k].cpu().numpy(), expect[k].cpu().numpy()) <= 1e-6, k
            assert cases.rel_err(g2[k].cpu().numpy(), ref_g[k].cpu().numpy()) <= 2e-6, k
    finally:
        lib.b200_wn_batch_mode(0)


def test_axpby_rows_matches_per_sample_loop(lib, orc):
    import torch
    rng = np.random.default_rng(51)
    rows, dim = 37, 784
    a = rng.standard_normal((rows, dim), dtype=np.float32); b = rng.standard_normal((rows, dim), dtype=np.float32)
    wa = rng.standard_normal(rows, dtype=np.float32); wb = rng.standard_normal(rows, dtype=np.float32)
    ta, tb, twa, twb = _t(a), _t(b), _t(wa), _t(wb)
    out = torch.empty_like(ta)
    lib.launch_axpby_rows(_pp(out), _pp(ta), _pp(tb), _pp(twa), _pp(twb), rows, dim, _st())
    loop = torch.empty_like(ta)
    for r in range(rows):  # what diffusion/edm.c:56-58 does
        lib.launch_weighted_sum(_pp(loop, r * dim), _pp(ta, r * dim), _pp(tb, r * dim), ctypes.c_float(float(wa[r])),
                                ctypes.c_float(float(wb[r])), dim, _st())
    torch.cuda.synchronize()
    assert torch.equal(out, loop)
    assert cases.rel_err(out.cpu().numpy(), orc.axpby_rows(a, b, wa, wb)) <= 1e-6


def test_no_bounded_wait_ran_out(lib):
    assert lib.b200_device_error_status() == 0
    assert lib.b200_launch_count() > 0


_GN_PATH_PIPELINED, _GN_PATH_DEEP, _GN_PATH_ONE_BARRIER = 1, 2, 3


@pytest.mark.parametrize("deep", [1, 0])
@pytest.mark.parametrize("shape", [dict(B=640, HW=1024, C=32, G=4), dict(B=1300, HW=400, C=16, G=2)])
def test_groupnorm_deep_staged_strips(lib, orc, shape, deep):
    """Enough strips per CTA (>= 8) that the deep-staged kernels are taken when asked for: full strips
    (1024 rows fill every register slot) and ragged ones (400 rows); same results, bit-reproducible, with the
    plain pipeline as the control."""
    p = dict(shape, act="silu")
    inp = cases.make_inputs("groupnorm", p, seed=43)
    ref = cases.oracle_run(orc, "groupnorm", p, inp)
    lib.b200_tune_set(b"gn_one_barrier", 0)  # the one-barrier strips would take these shapes first
    lib.b200_tune_set(b"gn_deep", deep)
    before = lib.b200_groupnorm_path_count(_GN_PATH_DEEP), lib.b200_groupnorm_path_count(_GN_PATH_PIPELINED)
    try:
        got = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
        got2 = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    finally:
        lib.b200_tune_set(b"gn_one_barrier", 1)
        lib.b200_tune_set(b"gn_deep", 1)
    taken = (lib.b200_groupnorm_path_count(_GN_PATH_DEEP) - before[0],
             lib.b200_groupnorm_path_count(_GN_PATH_PIPELINED) - before[1])
    assert taken == ((2, 2) if deep else (0, 4)), taken  # only the backward has a deep-staged form
    _check(got, ref, f"deep={deep}")
    for k in got:
        assert np.array_equal(got[k], got2[k]), k


# (B, HW, C, G): channels per group 8, 2, 4, 16, 2 and 8 -- one group per float4 column with 2, 1 and 4
# columns per group, and two groups per column; rows that fill every register slot (1024, 256) and ragged ones
_ONE_BARRIER_SHAPES = [dict(B=640, HW=1024, C=32, G=4), dict(B=700, HW=784, C=64, G=32), dict(B=1300, HW=256, C=32, G=8),
                       dict(B=600, HW=400, C=64, G=4), dict(B=1300, HW=1024, C=16, G=8),
                       dict(B=320, HW=1024, C=128, G=16)]  # the last one: forward in clusters of 4 CTAs


@pytest.mark.parametrize("act", ["silu", None, "mp_silu"])
@pytest.mark.parametrize("shape", _ONE_BARRIER_SHAPES)
def test_groupnorm_one_barrier_strips(lib, orc, shape, act):
    """The one-barrier strips are the default for these shapes (many strips per CTA, whole groups per float4
    column or two groups per column); checked against the oracle, for bit-reproducibility, and against the
    three-barrier pipelines on the same inputs."""
    p = dict(shape, act=act)
    inp = cases.make_inputs("groupnorm", p, seed=47)
    ref = cases.oracle_run(orc, "groupnorm", p, inp)
    before = lib.b200_groupnorm_path_count(_GN_PATH_ONE_BARRIER)
    got = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    got2 = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    assert lib.b200_groupnorm_path_count(_GN_PATH_ONE_BARRIER) - before == 4, "forward and backward, twice"
    lib.b200_tune_set(b"gn_one_barrier", 0)
    try:
        old = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    finally:
        lib.b200_tune_set(b"gn_one_barrier", 1)
    assert lib.b200_groupnorm_path_count(_GN_PATH_ONE_BARRIER) - before == 4
    _check(got, ref, f"one barrier {shape} {act}")
    for k in got:
        assert np.array_equal(got[k], got2[k]), k
        tol = cases.TOL_FWD if k in ("y", "mu", "rstd") else cases.TOL_BWD
        assert cases.rel_err(got[k], old[k]) <= tol, (k, cases.rel_err(got[k], old[k]))


@pytest.mark.parametrize("act", ["silu", None])
@pytest.mark.parametrize("shape", [_ONE_BARRIER_SHAPES[i] for i in (0, 1, 2, 4, 5)])  # the shapes with whole strips
def test_groupnorm_backward_tma_staging(lib, orc, shape, act):
    """The backward one-barrier strips with TMA staging (on request: one box per warp, tensor and strip, per-warp
    mbarriers with bounded waits): same results as the oracle and as the cp.async staging, bit-reproducible, and
    no wait ran out (the device error word stays 0)."""
    p = dict(shape, act=act)
    inp = cases.make_inputs("groupnorm", p, seed=53)
    ref = cases.oracle_run(orc, "groupnorm", p, inp)
    plain = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    before = lib.b200_groupnorm_path_count(_GN_PATH_ONE_BARRIER)
    lib.b200_tune_set(b"gn_bwd_tma", 2)
    try:
        got = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
        got2 = cases.gpu_run(lib, "groupnorm", p, inp, fused=True)
    finally:
        lib.b200_tune_set(b"gn_bwd_tma", 0)
    assert lib.b200_groupnorm_path_count(_GN_PATH_ONE_BARRIER) - before == 4
    assert lib.b200_device_error_status() == 0
    _check(got, ref, f"tma staging {shape} {act}")
    for k in got:
        assert np.array_equal(got[k], got2[k]), k
        tol = cases.TOL_FWD if k in ("y", "mu", "rstd") else cases.TOL_BWD
        assert cases.rel_err(got[k], plain[k]) <= tol, (k, cases.rel_err(got[k], plain[k]))
