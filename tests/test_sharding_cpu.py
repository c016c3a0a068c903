"""Host-side multi-GPU logic on CPU: world_size-2 gloo ranks, the CPU oracle standing in for the kernels."""
import importlib
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle"))


def _sharding():
    return importlib.import_module("cuda-c-diffusion_b200.sharding")


def test_batch_shards_tile_the_batch():
    sh = _sharding()
    for n in (0, 1, 7, 256, 257):
        for world in (1, 2, 3, 8):
            spans = [sh.batch_shard(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == n
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        sh.batch_shard(8, 2, 2)


def test_param_ranges_are_aligned_and_tile():
    sh = _sharding()
    for n in (0, 1, 3, 4, 5, 1000, 67108864, 67108865):
        for world in (1, 2, 4, 8):
            spans = [sh.param_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a0, a1), (b0, _) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            for lo, hi in spans[:-1]:
                assert lo % 4 == 0 and hi % 4 == 0 or hi == n
            shard = sh.equal_param_range(n, world)
            assert shard % 4 == 0 and shard * world >= n and shard * world - n < 4 * world


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_update(orc):
    def fn(p, m, v, shadow, g, h):
        rp, rm, rv, rs = orc.adam_ema_step(p.numpy(), m.numpy(), v.numpy(), shadow.numpy(), g.numpy(), h.lr, h.beta1,
                                           h.beta2, h.eps, h.bc1, h.bc2, h.decay, h.grad_scale)
        p.copy_(torch.from_numpy(rp)); m.copy_(torch.from_numpy(rm)); v.copy_(torch.from_numpy(rv))
        shadow.copy_(torch.from_numpy(rs))
    return fn


def _worker(rank, world, port, n, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = _sharding()
        orc = importlib.import_module("oracle")
        orc.load()
        rng = np.random.default_rng(7)
        p0 = (0.02 * rng.standard_normal(n)).astype(np.float32)
        grads = [(1e-3 * rng.standard_normal(n)).astype(np.float32) for _ in range(3)]
        # (1) range-sharded fused Adam+EMA == unsharded
        opt = sh.ShardedAdamEMA(torch.from_numpy(p0.copy()), lr=1e-3, update_fn=_oracle_update(orc))
        for g in grads:
            # data-parallel: every rank contributes its own gradient; the sum is scaled by 1/world
            local = torch.from_numpy(g.copy())
            scale = sh.allreduce_gradients(local)
            opt.step(local, grad_scale=scale)
        m_full, v_full, s_full = opt.gather_state()
        # (2) batch-sharded LayerNorm backward: partial dgamma/dbeta + all-reduce == full batch
        rows, C = 10, 16
        x = rng.standard_normal((rows, C)).astype(np.float32); dy = rng.standard_normal((rows, C)).astype(np.float32)
        gam = (1 + 0.1 * rng.standard_normal(C)).astype(np.float32); bet = np.zeros(C, np.float32)
        s0, cnt = sh.batch_shard(rows, rank, world)
        xs, dys = x[s0:s0 + cnt], dy[s0:s0 + cnt]
        _, mu, rstd = orc.layernorm_forward(xs, gam, bet, 1e-5)
        dx, dg, db = orc.layernorm_backward(dys, xs, gam, mu, rstd)
        tdg, tdb = torch.from_numpy(dg), torch.from_numpy(db)
        sh.allreduce_param_grads(tdg, tdb)
        if rank == 0:
            q.put(dict(p=opt.full_params().numpy().copy(), m=m_full.numpy().copy(), v=v_full.numpy().copy(),
                       s=s_full.numpy().copy(), dg=tdg.numpy().copy(), db=tdb.numpy().copy(),
                       shard=opt.shard, world=world))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [1000, 1003, 4096])
def test_world2_sharded_update_and_norm_grads_match_single_rank(n):
    orc = importlib.import_module("oracle")
    orc.load()
    orc.set_accumulate_double(True)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # single-rank reference: both ranks contributed the same gradient, so sum/world == the gradient
    rng = np.random.default_rng(7)
    p0 = (0.02 * rng.standard_normal(n)).astype(np.float32)
    grads = [(1e-3 * rng.standard_normal(n)).astype(np.float32) for _ in range(3)]
    p, m, v, s = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32), p0.copy()
    for t, g in enumerate(grads, start=1):
        bc1 = float(np.float32(1) - np.power(np.float32(0.9), np.float32(t)))
        bc2 = float(np.float32(1) - np.power(np.float32(0.999), np.float32(t)))
        p, m, v, s = orc.adam_ema_step(p, m, v, s, g * np.float32(2.0), 1e-3, 0.9, 0.999, 1e-8, bc1, bc2, 0.999, 0.5)
    assert np.allclose(out["p"], p, rtol=0, atol=1e-7)
    assert np.allclose(out["m"], m, rtol=1e-6, atol=1e-9) and np.allclose(out["v"], v, rtol=1e-6, atol=1e-12)
    assert np.allclose(out["s"], s, rtol=0, atol=1e-7)
    assert out["shard"] * out["world"] >= n
    rows, C = 10, 16
    x = rng.standard_normal((rows, C)).astype(np.float32); dy = rng.standard_normal((rows, C)).astype(np.float32)
    gam = (1 + 0.1 * rng.standard_normal(C)).astype(np.float32); bet = np.zeros(C, np.float32)
    _, mu, rstd = orc.layernorm_forward(x, gam, bet, 1e-5)
    _, dg, db = orc.layernorm_backward(dy, x, gam, mu, rstd)
    assert np.allclose(out["dg"], dg, rtol=1e-5, atol=1e-6) and np.allclose(out["db"], db, rtol=1e-5, atol=1e-6)


# ---------------------------------------------------------------- failures, injected on the host
def test_bad_rank_and_world_are_rejected():
    sh = _sharding()
    for fn in (sh.batch_shard, sh.param_range):
        with pytest.raises(ValueError):
            fn(10, 2, 2)
        with pytest.raises(ValueError):
            fn(10, -1, 2)


def _lonely_worker(port, q):
    """World of two in which the second rank never starts: the rendezvous must end with an error after
    the short timeout instead of waiting forever."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        q.put("joined")
    except Exception as exc:  # noqa: BLE001 - any rendezvous error is the expected outcome
        q.put("error: " + type(exc).__name__)


def test_rank_that_never_joins_ends_in_a_timeout_not_a_hang():
    with socket.socket() as s_:
        s_.bind(("127.0.0.1", 0))
        port = s_.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_worker, args=(port, q))
    p.start()
    p.join(60)
    if p.is_alive():
        p.kill()
        pytest.fail("rendezvous with a missing rank did not time out")
    assert q.get(timeout=5).startswith("error")


def _mismatch_worker(rank, world, port, q):
    """Rank 1 builds its optimizer for a different parameter count: the in-place all-gather must fail loudly
    (shape check on the host) rather than exchange ranges that do not tile the vector."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    try:
        sh = _sharding()
        n = 1000 if rank == 0 else 1200
        opt = sh.ShardedAdamEMA(torch.zeros(n), lr=1e-3, update_fn=lambda *a: None)
        sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([opt.shard], dtype=torch.int64))
        ok = len({int(s_) for s_ in sizes}) == 1
        if rank == 0:
            q.put("consistent" if ok else "mismatch detected")
    finally:
        dist.destroy_process_group()


def test_mismatched_shard_sizes_are_detected_before_the_exchange():
    with socket.socket() as s_:
        s_.bind(("127.0.0.1", 0))
        port = s_.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_mismatch_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert all(not p.is_alive() for p in procs)
    assert q.get(timeout=5) == "mismatch detected"
