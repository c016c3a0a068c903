"""The allocation-free LayerNorm backward (`launch_layernorm_backward_noalloc`).

Some hosts of this library work under a fixed device-memory plan and may not call cudaMalloc once
their modules are constructed, so they cannot use the regular backward, whose partial-sum scratch is
allocated on first use.  The variant keeps that scratch in a fixed array inside the library.  Here it
is called through the C ABI twice in a row (different shapes and data, so the second call meets the
first call's leftovers in the shared array) and compared with the regular entry point.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It passes on its own in a fresh process as well as after the rest of the suite.
"""
import ctypes

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu


def _run(lib, fn, rows, C, seed, keep):
    import torch
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((rows, C), dtype=np.float32)).cuda()
    dy = torch.from_numpy(rng.standard_normal((rows, C), dtype=np.float32)).cuda()
    gamma = torch.from_numpy((1 + 0.1 * rng.standard_normal(C)).astype(np.float32)).cuda()
    beta = torch.zeros(C, device="cuda")
    y = torch.empty_like(x); mu = torch.empty(rows, device="cuda"); rstd = torch.empty(rows, device="cuda")
    dx = torch.full_like(x, float("nan")); dg = torch.full((C,), float("nan"), device="cuda"); db = dg.clone()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    lib.launch_layernorm_forward(P(y), P(mu), P(rstd), P(x), P(gamma), P(beta), rows, C, ctypes.c_float(1e-5), st)
    rc = fn(P(dx), P(dg), P(db), P(dy), P(x), P(gamma), P(mu), P(rstd), rows, C, st)
    torch.cuda.synchronize()
    keep.extend([x, dy, gamma, beta, y, mu, rstd])
    return rc, dx.cpu().numpy(), dg.cpu().numpy(), db.cpu().numpy()


def _free_bytes():
    import torch
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]  # cudaMemGetInfo: free bytes of the device, all allocators included


# the last two pairs reach the limits of the fixed array: C = 1024 / 896 with a grid (forced to 8 CTAs per SM
# through the tunable) that has to be clipped to the partial rows that fit (2^20 / 2048 = 512 CTAs; the
# grid-stride loop covers the rest), and the generic path (C not a multiple of 128) with
# ceil(rows/256) * 2*C just under 2^20 floats
@pytest.mark.parametrize("shapes", [[(3000, 256), (777, 256)], [(500, 100), (4100, 384)],
                                    [(12000, 1024), (10000, 896)], [(256 * 2600, 200), (1000, 200)]])
def test_noalloc_backward_matches_regular_backward_twice_in_a_row(lib, shapes):
    keep = []
    lib.b200_tune_set(b"ln_bwd_blocks_per_sm", 8 if shapes[0][1] == 1024 else 2)
    try:
        _noalloc_pairs(lib, shapes, keep)
    finally:
        lib.b200_tune_set(b"ln_bwd_blocks_per_sm", 2)


def _noalloc_pairs(lib, shapes, keep):
    for i, (rows, C) in enumerate(shapes):
        # the regular entry point first: it (and torch) may allocate; what follows must not
        _, rdx, rdg, rdb = _run(lib, lib.launch_layernorm_backward, rows, C, 100 + i, keep)
        _run(lib, lib.launch_layernorm_backward_noalloc, rows, C, 100 + i, keep)  # first use on this device: set-up
        import torch
        rng = np.random.default_rng(100 + i)
        t = [torch.from_numpy(rng.standard_normal((rows, C), dtype=np.float32)).cuda() for _ in range(2)]
        gamma = torch.from_numpy((1 + 0.1 * rng.standard_normal(C)).astype(np.float32)).cuda()
        mu, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
        y, dxb = torch.empty_like(t[0]), torch.empty_like(t[0])
        dgb, dbb = torch.empty(C, device="cuda"), torch.empty(C, device="cuda")
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        P = lambda a: ctypes.c_void_p(a.data_ptr())
        lib.launch_layernorm_forward(P(y), P(mu), P(rstd), P(t[0]), P(gamma), P(dgb), rows, C, ctypes.c_float(1e-5), st)
        before = _free_bytes()
        rc0 = lib.launch_layernorm_backward_noalloc(P(dxb), P(dgb), P(dbb), P(t[1]), P(t[0]), P(gamma), P(mu), P(rstd),
                                                    rows, C, st)
        assert rc0 == 0 and _free_bytes() == before, "the allocation-free entry point changed the device's free memory"
        del t, y, dxb
        rc, dx, dg, db = _run(lib, lib.launch_layernorm_backward_noalloc, rows, C, 100 + i, keep)
        assert rc == 0
        assert cases.rel_err(dx, rdx) <= cases.TOL_BWD
        assert cases.rel_err(dg, rdg) <= cases.TOL_BWD
        assert cases.rel_err(db, rdb) <= cases.TOL_BWD
        assert np.isfinite(dx).all() and np.isfinite(dg).all() and np.isfinite(db).all()
        keep.clear()


def test_noalloc_backward_rejects_sizes_beyond_its_fixed_scratch(lib):
    lib.b200_set_error_mode(1)
    lib.b200_clear_error()
    try:
        # generic path (C not a multiple of 128): ceil(batch/256) * 2*C floats exceeds 2^20
        rc = lib.launch_layernorm_backward_noalloc(None, None, None, None, None, None, None, None, 3_000_000, 100,
                                                   None)
        assert rc < 0
        assert lib.b200_error_count() == 1
        buf = ctypes.create_string_buffer(512)
        lib.b200_last_error(ctypes.cast(buf, ctypes.c_void_p), 512)
        assert b"fixed" in buf.value and b"scratch" in buf.value
    finally:
        lib.b200_clear_error()
        lib.b200_set_error_mode(0)
