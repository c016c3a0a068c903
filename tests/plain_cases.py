"""Table-driven cases for the launchers of the reference C ABI that sit either side of the
fused layer kernels in a training step (im2col/col2im, resampling, attention glue, FiLM,
bias and loss helpers; reference src/kernels.cu:95-161 and :750-1313).

One case = one launcher call.  The same argument list drives three implementations:

* `run_oracle`  -- oracle/layer_oracle.c through `oracle.raw`,
* `run_gpu`     -- any CUDA library that exports the reference's launcher set (this
                   repository's, or the reference's own kernels.cu built for sm_100a).

Argument descriptors (device pointers in the C prototype):
    ("in",  key, shape[, scale])   seeded normal input
    ("arr", key, ndarray)          explicit input
    ("out", key, shape)            output written in full by the launcher
    ("acc", key, shape)            output the launcher accumulates into (starts at zero)
    ("io",  key, shape)            seeded input updated in place and returned
Plain python ints/floats are passed by value; `Long(n)` marks an extent that the oracle's
prototype declares as `long` (the launchers take `int`).
"""
from __future__ import annotations

import ctypes

import numpy as np


class Long(int):
    pass


def _softmax_rows(x):
    e = np.exp(x - x.max(axis=1, keepdims=True))
    return (e / e.sum(axis=1, keepdims=True)).astype(np.float32)


def _conv(name, B, H, W, C, K, stride, pad):
    Ho, Wo = (H + 2 * pad - K) // stride + 1, (W + 2 * pad - K) // stride + 1
    dims = (B, H, W, C, K, stride, pad, Ho, Wo)
    return [
        (f"im2col_{name}", "im2col", [("out", "col", (B * Ho * Wo, K * K * C)), ("in", "im", (B, H, W, C)), *dims], 0.0),
        (f"col2im_{name}", "col2im", [("acc", "gim", (B, H, W, C)), ("in", "gcol", (B * Ho * Wo, K * K * C)), *dims], 1e-6),
    ]


def _resample(name, B, H, W, C):
    return [
        (f"avg_pool_{name}", "avg_pool_2x", [("out", "y", (B, H // 2, W // 2, C)), ("in", "x", (B, H, W, C)), B, H, W, C], 1e-6),
        (f"avg_pool_bwd_{name}", "avg_pool_2x_backward",
         [("acc", "gx", (B, H, W, C)), ("in", "gy", (B, H // 2, W // 2, C)), B, H, W, C], 0.0),
        (f"upsample_{name}", "nearest_upsample_2x", [("out", "y", (B, 2 * H, 2 * W, C)), ("in", "x", (B, H, W, C)), B, H, W, C], 0.0),
        (f"upsample_bwd_{name}", "nearest_upsample_2x_backward",
         [("out", "gx", (B, H, W, C)), ("in", "gy", (B, 2 * H, 2 * W, C)), B, H, W, C], 1e-6),
    ]


def _film(name, B, H, W, C):
    return [
        (f"film_{name}", "spatial_modulate", [("out", "y", (B, H, W, C)), ("in", "x", (B, H, W, C)), ("in", "cond", (B, C)), B, H, W, C], 1e-6),
        (f"film_bwd_{name}", "spatial_modulate_backward",
         [("out", "gx", (B, H, W, C)), ("out", "gcond", (B, C)), ("in", "g", (B, H, W, C)), ("in", "x", (B, H, W, C)),
          ("in", "cond", (B, C)), B, H, W, C], 1e-4),
        (f"spatial_add_{name}", "spatial_add", [("io", "x", (B, H, W, C)), ("in", "bias", (B, C)), B, H, W, C], 1e-6),
        (f"spatial_sum_{name}", "spatial_reduce_sum", [("out", "s", (B, C)), ("in", "x", (B, H * W, C)), B, H * W, C], 1e-5),
    ]


def _build():
    rng = np.random.default_rng(99)
    cs = []
    cs += _conv("3x3_c4", 2, 6, 5, 4, 3, 1, 1)
    cs += _conv("1x1_c3", 2, 6, 5, 3, 1, 1, 0)
    cs += _conv("3x3s2_c16", 2, 6, 5, 16, 3, 2, 1)
    cs += _conv("5x5_c3", 1, 7, 6, 3, 5, 1, 2)
    cs += _conv("3x3_c16_14", 2, 14, 14, 16, 3, 1, 1)
    cs += _resample("c8", 2, 6, 4, 8)
    cs += _resample("c5", 2, 6, 4, 5)
    cs += _resample("c16_14", 2, 14, 14, 16)
    x = (3 * rng.standard_normal((37, 49))).astype(np.float32)
    cs += [
        ("attn_softmax_49", "attn_softmax", [("out", "p", (37, 49)), ("arr", "x", x), 37, 49], 1e-5),
        ("attn_softmax_inplace", "attn_softmax", [("io", "x", (41, 196)), ("alias", "x"), 41, 196], 1e-5),
        ("attn_softmax_bwd_49", "attn_softmax_backward",
         [("out", "gx", (37, 49)), ("in", "g", (37, 49)), ("arr", "p", _softmax_rows(x)), 37, 49], 1e-4),
        ("permute_d8", "permute_0213", [("out", "y", (2, 4, 5, 8)), ("in", "x", (2, 5, 4, 8)), 2, 5, 4, 8], 0.0),
        ("permute_d3", "permute_0213", [("out", "y", (2, 4, 5, 3)), ("in", "x", (2, 5, 4, 3)), 2, 5, 4, 3], 0.0),
        ("permute_attn", "permute_0213", [("out", "y", (4, 1, 49, 128)), ("in", "x", (4, 49, 1, 128)), 4, 49, 1, 128], 0.0),
    ]
    cs += _film("c64_7", 3, 7, 7, 64)
    cs += _film("c6_7", 3, 7, 7, 6)
    cs += _film("c32_28", 2, 28, 28, 32)
    tg = rng.integers(0, 10, 6).astype(np.int32)
    idx = np.array([0, 3, 3, 6, 9, -2, 1, 1, 1], np.float32)  # out-of-range rows are clamped
    cs += [
        ("add_bias", "add_bias", [("io", "Y", (9, 12)), ("in", "b", (12,)), 9, 12], 1e-6),
        ("bias_grad", "bias_grad", [("out", "gb", (12,)), ("in", "g", (9, 12)), 9, 12], 1e-5),
        ("bias_grad_tall", "bias_grad", [("out", "gb", (128,)), ("in", "g", (6272, 128)), 6272, 128], 1e-5),
        ("bias_grad_odd", "bias_grad", [("out", "gb", (37,)), ("in", "g", (1000, 37)), 1000, 37], 1e-5),
        ("mse", "mse_fwd_bwd", [("out", "grad", (5, 784)), ("out", "loss", (5,)), ("in", "pred", (5, 784)),
                                ("in", "target", (5, 784)), 5, 784], 1e-5),
        ("softmax_xent", "softmax_xent", [("out", "gz", (6, 10)), ("out", "loss", (6,)), ("in", "z", (6, 10), 2.0),
                                          ("arr", "targets", tg), 6, 10], 1e-5),
        ("clamp", "clamp", [("io", "x", (1001,), 3.0), -1.0, 2.0, Long(1001)], 0.0),
        ("sgd", "sgd_step", [("io", "p", (777,)), ("in", "g", (777,)), 0.1, Long(777)], 1e-6),
        ("modulate", "modulate", [("out", "h2", (500,)), ("in", "h1", (500,)), ("in", "c", (500,)), Long(500)], 1e-6),
        ("modulate_bwd", "modulate_backward", [("out", "gh1", (500,)), ("out", "gc", (500,)), ("in", "gh2", (500,)),
                                               ("in", "h1", (500,)), ("in", "c", (500,)), Long(500)], 1e-6),
        ("embed_gather", "embed_gather", [("out", "y", (9, 12)), ("in", "table", (7, 12)), ("arr", "idx", idx), 9, 12, 7], 0.0),
        ("embed_scatter", "embed_scatter", [("acc", "gt", (7, 12)), ("in", "g", (9, 12)), ("arr", "idx", idx), 9, 12, 7], 1e-5),
        ("channel_cat", "channel_cat", [("out", "y", (41, 96)), ("in", "a", (41, 64)), ("in", "b", (41, 32)), Long(41), 64, 32], 0.0),
        ("channel_cat_odd", "channel_cat", [("out", "y", (41, 8)), ("in", "a", (41, 5)), ("in", "b", (41, 3)), Long(41), 5, 3], 0.0),
        ("channel_split", "channel_split", [("out", "ga", (41, 64)), ("out", "gb", (41, 32)), ("in", "g", (41, 96)), Long(41), 64, 32], 0.0),
        ("channel_split_odd", "channel_split", [("out", "ga", (41, 5)), ("out", "gb", (41, 3)), ("in", "g", (41, 8)), Long(41), 5, 3], 0.0),
    ]
    return cs


# (case name, launcher name without the `launch_` prefix, argument list, tolerance);
# tolerance 0.0 means bit-exact, otherwise max|a-b| / max|ref|.
PLAIN_CASES = _build()


def seed_of(name):
    return 7 + sum((i + 1) * ord(ch) for i, ch in enumerate(name)) % (2 ** 31)


def materialise(name, args):
    """Host arrays for every pointer argument, in order; returns (arrays, returned keys)."""
    rng = np.random.default_rng(seed_of(name))
    arrays, returned = {}, []
    for a in args:
        if not isinstance(a, tuple):
            continue
        kind, key = a[0], a[1]
        if kind == "in" or kind == "io":
            if key not in arrays:
                scale = a[3] if len(a) > 3 else 1.0
                arrays[key] = (np.float32(scale) * rng.standard_normal(a[2], dtype=np.float32)).astype(np.float32)
            if kind == "io":
                returned.append(key)
        elif kind == "arr":
            arrays[key] = np.ascontiguousarray(a[2])
        elif kind in ("out", "acc"):
            arrays[key] = np.zeros(a[2], np.float32)
            returned.append(key)
        elif kind == "alias":
            pass
        else:
            raise KeyError(kind)
    return arrays, returned


def run_oracle(orc, name, fn, args):
    arrays, returned = materialise(name, args)
    call = []
    for a in args:
        if isinstance(a, tuple):
            call.append(arrays[a[1]])
        elif isinstance(a, Long):
            call.append(orc.L(int(a)))
        else:
            call.append(a)
    orc.raw(fn, *call)
    return {k: arrays[k] for k in returned}


def run_gpu(lib, name, fn, args):
    import torch

    arrays, returned = materialise(name, args)
    dev = {k: torch.from_numpy(v).cuda() for k, v in arrays.items()}
    call = []
    for a in args:
        if isinstance(a, tuple):
            call.append(ctypes.c_void_p(dev[a[1]].data_ptr()))
        elif isinstance(a, float):
            call.append(ctypes.c_float(a))
        else:
            call.append(int(a))
    getattr(lib, "launch_" + fn)(*call, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return {k: dev[k].cpu().numpy() for k in returned}


def compare(got, ref, tol, label):
    for k, r in ref.items():
        g = got[k]
        if tol == 0.0:
            assert np.array_equal(g, r), f"{label}:{k} is not bit-identical"
        else:
            scale = max(float(np.max(np.abs(r))) if r.size else 0.0, 1e-6)
            err = float(np.max(np.abs(g.astype(np.float64) - r.astype(np.float64)))) / scale if r.size else 0.0
            assert err <= tol, f"{label}:{k} rel err {err:.3e} > {tol:.0e}"
