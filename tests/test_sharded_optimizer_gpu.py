"""GPU: the range-sharded fused Adam+EMA (csrc/host/b200_sharded_optimizer.c, C + NCCL + CUDA IPC) and the two
launchers under it (launch_adam_ema_step_bcast, launch_copy_multi).

One GPU is enough for the kernels, the flat path with world = 1, the checkpoint round trip and the host-side
failure forms; the exchange between ranks (in-place all-gather, and peer stores fused into the update kernel)
runs as child processes on 2 GPUs where they are available, with NVLS off and plain peer stores."""
import ctypes
import json
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "cuda-c-diffusion_b200" / "build" / "bin"
F = ctypes.c_float


def _need(exe):
    if not exe.exists():
        pytest.skip(f"{exe.name} not built (needs the reference sources at build time)")
    return exe


def _two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")


def _ranks(exe, args, world, tmp_path, per_rank_args=None, env_extra=None, timeout=180):
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), NCCL_NVLS_ENABLE="0",
                   **(env_extra or {}))
        extra = (per_rank_args or {}).get(r, [])
        procs.append(subprocess.Popen([str(exe), *args, *extra, "--id-file", str(tmp_path / "nccl.id")], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    try:
        outs = [p.communicate(timeout=timeout) for p in procs]
    except subprocess.TimeoutExpired:
        for p in procs:
            p.kill()
        pytest.fail(f"ranks did not finish within {timeout} s")
    return procs, outs


def test_update_with_extra_destinations_equals_the_plain_update(lib, capi):
    """launch_adam_ema_step_bcast with two further destination buffers (on the same GPU here; peer pointers
    in the sharded optimizer): p, m, v, shadow bit-identical to launch_adam_ema_step, destinations equal p."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(5)
    n = 4 * 250_003
    p0 = 0.02 * torch.randn(n, device="cuda", generator=g)
    grad = 1e-3 * torch.randn(n, device="cuda", generator=g)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    hp = (F(1e-4), F(0.9), F(0.999), F(1e-8), F(0.1), F(0.001), F(0.999), F(0.5))
    a = [p0.clone(), torch.zeros_like(p0), torch.zeros_like(p0), p0.clone()]
    b = [x.clone() for x in a]
    d1, d2 = torch.zeros(n + 8, device="cuda"), torch.zeros(n, device="cuda")
    lib.launch_adam_ema_step(*(P(t) for t in a), P(grad), *hp, ctypes.c_longlong(n), st)
    peers = capi.PeerDests()
    peers.dst[0], peers.dst[1], peers.count = d1.data_ptr() + 16, d2.data_ptr(), 2
    lib.launch_adam_ema_step_bcast(*(P(t) for t in b), P(grad), ctypes.byref(peers), *hp, ctypes.c_longlong(n), st)
    torch.cuda.synchronize()
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    assert torch.equal(d1[4:4 + n], b[0]) and torch.equal(d2, b[0])
    assert float(d1[:4].abs().sum()) == 0 and float(d1[4 + n:].abs().sum()) == 0
    # an unaligned destination and a length that is not a multiple of 4 are rejected on the host
    lib.b200_set_error_mode(1)
    lib.b200_clear_error()
    try:
        peers.dst[0] = d1.data_ptr() + 4
        lib.launch_adam_ema_step_bcast(*(P(t) for t in b), P(grad), ctypes.byref(peers), *hp, ctypes.c_longlong(n), st)
        lib.launch_adam_ema_step_bcast(*(P(t) for t in b), P(grad), ctypes.byref(peers), *hp, ctypes.c_longlong(n - 1), st)
        assert lib.b200_error_count() == 2
    finally:
        lib.b200_clear_error()
        lib.b200_set_error_mode(0)


def test_copy_multi_packs_and_unpacks_a_parameter_list(lib, capi):
    import torch
    rng = np.random.default_rng(9)
    sizes = [1, 7, 4096, 1, 73728, 0, 128, 3, 36864] * 9  # 81 items: more than one table
    src = [torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda() for n in sizes]
    offs, total = [], 0
    for n in sizes:
        offs.append(total)
        total += (n + 3) // 4 * 4
    flat = torch.full((total,), -1.0, device="cuda")
    items = (capi.CopyItem * len(sizes))()
    for i, n in enumerate(sizes):
        items[i] = capi.CopyItem(flat.data_ptr() + 4 * offs[i], src[i].data_ptr(), n)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    lib.launch_copy_multi(ctypes.cast(items, ctypes.c_void_p), len(sizes), st)
    back = [torch.zeros_like(t) for t in src]
    for i, n in enumerate(sizes):
        items[i] = capi.CopyItem(back[i].data_ptr(), flat.data_ptr() + 4 * offs[i], n)
    lib.launch_copy_multi(ctypes.cast(items, ctypes.c_void_p), len(sizes), st)
    torch.cuda.synchronize()
    for a, b in zip(src, back):
        assert torch.equal(a, b)
    keep = torch.ones(total, dtype=torch.bool)
    for o, n in zip(offs, sizes):
        keep[o:o + n] = False
    assert bool((flat.cpu()[keep] == -1.0).all()), "padding between tensors must stay untouched"


@pytest.mark.parametrize("n", [67_108_864 // 16, 1_000_003])
def test_flat_sharded_optimizer_on_one_rank(tmp_path, n):
    """world = 1: both exchange forms degenerate to the plain fused update; bit-identical to it over three
    steps, and the sharded state survives a round trip through the reference's training checkpoint."""
    exe = _need(BIN / "sharded_adam_bench")
    res = subprocess.run([str(exe), "--params", str(n), "--iters", "2", "--warmup", "1", "--check", "--ckpt",
                          str(tmp_path / "state.ckpt")], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    got = json.loads(next(ln for ln in res.stdout.splitlines() if ln.startswith("{")))["sharded_adam_ema"]
    assert got["checked"] is True and got["failures"] == 0 and got["params"] == n


def test_flat_sharded_optimizer_on_two_ranks(tmp_path):
    """2 GPUs: update + in-place all-gather and update-with-peer-stores both leave every rank with exactly the
    parameters of an unsharded update; checkpoint round trip of the gathered state."""
    _two_gpus()
    exe = _need(BIN / "sharded_adam_bench")
    procs, outs = _ranks(exe, ["--params", "4000003", "--iters", "3", "--warmup", "2", "--check", "--ckpt",
                               str(tmp_path / "state.ckpt")], 2, tmp_path)
    assert all(p.returncode == 0 for p in procs), outs
    got = json.loads(next(ln for ln in outs[0][0].splitlines() if ln.startswith("{")))["sharded_adam_ema"]
    assert got["n_gpus"] == 2 and got["failures"] == 0 and got["shard"] * 2 >= 4000003


def test_rank_built_for_another_model_is_caught_before_any_exchange(tmp_path):
    """Failure injected on the host: rank 1 is started with a different parameter count.  Every rank sees the
    mismatch in the (total, shard, world) triples it gathers at creation and gives up with a message; no
    collective ever runs on buffers of different sizes."""
    _two_gpus()
    exe = _need(BIN / "sharded_adam_bench")
    procs, outs = _ranks(exe, ["--iters", "1", "--warmup", "1"], 2, tmp_path,
                         per_rank_args={0: ["--params", "1000000"], 1: ["--params", "1000004"]})
    assert all(p.returncode != 0 for p in procs), outs
    assert "reports" in outs[0][1] and "reports" in outs[1][1]


def test_missing_peer_ends_with_an_error_not_a_hang(tmp_path):
    """Rank 1 of a world of two starts alone: the NCCL id never appears, the bounded host-side wait runs out."""
    exe = _need(BIN / "sharded_adam_bench")
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="0", B200_ID_WAIT_S="1.5")
    res = subprocess.run([str(exe), "--params", "1000", "--id-file", str(tmp_path / "never")], env=env,
                         capture_output=True, text=True, timeout=120)
    assert res.returncode != 0 and "did not publish the NCCL id" in res.stderr


def _dump(exe, tmp_path, name, extra, world=1):
    dump = tmp_path / f"{name}.bin"
    args = ["--fp32", "--steps", "3", "--warmup", "2", "--batch", "16", "--dump", str(dump), *extra]
    if world == 1:
        res = subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    else:
        (tmp_path / name).mkdir()
        procs, outs = _ranks(exe, args, world, tmp_path / name)
        assert all(p.returncode == 0 for p in procs), outs
    return np.fromfile(dump, dtype=np.float32)


def test_edm_trainer_with_sharded_optimizer_matches_replicated_on_one_rank(tmp_path):
    """edm_dp_train --sharded: gradients packed into the flat arena, fused update of the (whole) range,
    parameters unpacked -- same loss and parameters as the replicated multi-tensor update."""
    exe = _need(BIN / "edm_dp_train_fastconv")
    a = _dump(exe, tmp_path, "replicated", [])
    b = _dump(exe, tmp_path, "sharded", ["--sharded", "allgather"])
    assert a.size == b.size and a.size > 1_000_000
    assert abs(a[0] - b[0]) <= 1e-6 * abs(a[0])
    assert np.abs(a[1:] - b[1:]).max() <= 1e-6 * np.abs(a[1:]).max()


@pytest.mark.parametrize("how", ["allgather", "peer"])
def test_edm_trainer_with_sharded_optimizer_on_two_ranks(tmp_path, how):
    """2 GPUs: reduce-scatter + range-sharded update + exchange against all-reduce + replicated update from the
    same seeds (the two reductions add in different orders, hence a tolerance), and a sharded checkpoint written
    by `--save` loads back into a replicated run."""
    _two_gpus()
    exe = _need(BIN / "edm_dp_train_fastconv")
    a = _dump(exe, tmp_path, "replicated", [], world=2)
    ck = tmp_path / "sharded.ckpt"
    b = _dump(exe, tmp_path, "sharded", ["--sharded", how, "--save", str(ck)], world=2)
    assert abs(a[0] - b[0]) <= 1e-5 * abs(a[0])
    assert np.abs(a[1:] - b[1:]).max() <= 2e-5 * np.abs(a[1:]).max()
    # the file is the reference's per-tensor layout: a replicated single-rank run can resume from it
    res = subprocess.run([str(exe), "--fp32", "--batch", "8", "--resume", str(ck), "--warmup", "0", "--steps", "0",
                          "--dump", str(tmp_path / "resumed.bin")], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    c = np.fromfile(tmp_path / "resumed.bin", dtype=np.float32)
    assert np.array_equal(c[1:], b[1:])
