"""Which kernel family the GroupNorm dispatcher picks for a shape (`b200_groupnorm_describe`: walks the dispatcher
without a CUDA call, so these rules are checked on a CPU box; the SM count is taken as 148 there).

The expectations are the measured winners of each shape.  The sweep at the end guards a bug that was once in
the backward planner: for 16 x 16 and smaller samples with 128 channels and more it chose a 1024-thread CTA it
cannot run and fell through to the chunked kernels, 3.5 times slower.
"""
import ctypes
import importlib
import itertools
import re

import pytest

capi = importlib.import_module("cuda-c-diffusion_b200.capi")

NONE, RELU, SILU, MP_SILU = 0, 1, 3, 5


@pytest.fixture(scope="module")
def describe():
    lib = capi.load()
    buf = ctypes.create_string_buffer(256)

    def run(B, HW, C, G, act, backward):
        n = lib.b200_groupnorm_describe(B, HW, C, G, act, int(backward), ctypes.cast(buf, ctypes.c_void_p), 256)
        assert n > 0, (B, HW, C, G, act, backward)
        text = buf.value.decode()
        rec = dict(kv.split("=") for kv in text.split())
        return {k: (v if k == "family" else int(v)) for k, v in rec.items()}

    return run


CASES = [
    # B, HW, C, G, act, backward -> family, threads, strip channels, cluster width
    ((256, 1024, 256, 32, SILU, False), ("one-barrier", 1024, 32, 4)),   # the benchmark step: forward in clusters of 4
    ((256, 1024, 256, 32, SILU, True), ("one-barrier", 512, 16, 1)),
    ((256, 1024, 256, 32, NONE, False), ("one-barrier", 1024, 32, 4)),
    ((128, 1024, 256, 32, SILU, False), ("one-barrier", 1024, 32, 1)),   # 7 strips per CTA: too few for clusters
    ((128, 784, 64, 32, NONE, False), ("one-barrier", 448, 16, 1)),      # exact-fill CTAs, two groups per float4 column
    ((128, 784, 64, 32, NONE, True), ("pipelined", 512, 16, 1)),         # 4 strips per CTA: three-barrier kernel kept
    ((128, 784, 64, 32, SILU, True), ("pipelined", 448, 16, 1)),         # ... on exact-fill CTAs where an activation is paid for
    ((256, 784, 128, 32, SILU, False), ("one-barrier", 896, 32, 1)),
    ((256, 784, 128, 32, SILU, True), ("one-barrier", 448, 16, 1)),
    ((256, 196, 256, 32, SILU, False), ("one-barrier", 448, 64, 1)),
    ((256, 196, 256, 32, SILU, True), ("one-barrier", 448, 64, 1)),
    ((256, 256, 256, 32, SILU, True), ("one-barrier", 512, 64, 1)),
    ((32, 4096, 256, 32, SILU, False), ("chunked", 512, 16, 1)),         # 64 x 64 samples do not fit a CTA's registers
    ((32, 4096, 256, 32, SILU, True), ("chunked", 512, 16, 1)),
    ((3, 49, 64, 32, NONE, False), ("strip", 512, 64, 1)),               # fewer strips than CTA slots: one strip per CTA
    ((2, 15, 6, 3, NONE, False), ("generic", 256, 0, 1)),                # C not a multiple of 4
    ((256, 1024, 256, 32, RELU, False), ("generic", 256, 0, 1)),         # activations the strips do not instantiate
]


@pytest.mark.parametrize("shape,expected", CASES)
def test_dispatch_of_measured_shapes(describe, shape, expected):
    got = describe(*shape)
    assert (got["family"], got["threads"], got["strip_channels"], got["cluster"]) == expected, got


def test_bad_arguments_are_refused():
    lib = capi.load()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.b200_groupnorm_describe(4, 16, 30, 4, 0, 0, p, 64) == -1   # C not divisible by G
    assert lib.b200_groupnorm_describe(0, 16, 32, 4, 0, 0, p, 64) == -1
    assert lib.b200_groupnorm_describe(4, 16, 32, 4, 0, 0, None, 64) == -1


def test_register_resident_shapes_never_fall_to_the_chunked_or_generic_kernels(describe):
    """Every sample of at most 32 x 32 pixels with 32..512 channels in groups of 2..16 fits the register-resident
    strips, forward and backward, with and without activation."""
    bad = []
    for B, HW, C, cpg, act, bwd in itertools.product((32, 256), (16, 49, 64, 196, 256, 784, 1024), (32, 64, 128, 256, 512),
                                                     (2, 4, 8, 16), (NONE, SILU), (False, True)):
        got = describe(B, HW, C, C // cpg, act, bwd)
        if got["family"] in ("chunked", "generic"):
            bad.append(((B, HW, C, C // cpg, act, bwd), got["family"]))
    assert not bad, bad[:10]


def test_tma_staging_is_a_request_and_keeps_the_geometry(describe):
    """The backward's TMA staging is off by default; asked for, the dispatcher still plans the same one-barrier
    launch (same CTAs, strip width and shared memory), and planning encodes no tensor map (no driver call)."""
    lib = capi.load()
    shape = (256, 1024, 256, 32, SILU, True)
    plain = describe(*shape)
    lib.b200_tune_set(b"gn_bwd_tma", 2)
    try:
        asked = describe(*shape)
    finally:
        lib.b200_tune_set(b"gn_bwd_tma", 0)
    assert plain["family"] == "one-barrier" and asked == plain
