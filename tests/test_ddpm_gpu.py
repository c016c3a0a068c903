"""GPU: the DDPM half of the path, end to end through the reference's own trainer.

The reference's unmodified ddpm/main_ddpm.c + diffusion/ddpm.c + diffusion/train.c run a few fp32
training steps from a fixed seed and write the reference's own training checkpoint
(src/checkpoint.c: parameters, EMA shadows, Adam moments).  Three builds of that program:

  ddpm_demo_ref          reference host modules + reference kernels.cu           (oracle/_ref)
  ddpm_demo_b200         reference host modules + this library's kernels         (drop-in at the launch_* ABI)
  ddpm_demo_b200_fused   this repository's conv_residual / conv2d host modules   (GroupNorm+SiLU fused in the block)

The two builds on this library must agree with each other to fp32 round-off.  Against the reference's
kernels the comparison has a floor the reference sets itself: its GroupNorm kernels are racy on this GPU
(two block_reduce_sum calls without a barrier between them, src/kernels.cu:72-91,647-648), so two runs of
ddpm_demo_ref from the same seed differ; this library must be as close to each reference run as the
reference runs are to each other.
"""
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "cuda-c-diffusion_b200" / "build" / "bin"
REFBIN = ROOT / "oracle" / "_ref"

STEPS = 3
INI = """channels = 32,64,128
emb_dim = 64
heads = 4
num_groups = 32
batch_size = 16
train_steps = {steps}
lr = 1e-3
lr_warmup = 500
lr_ref = 2000
snr_gamma = 5.0
ema_decay = 0.999
T = 1000
beta_start = 1e-4
beta_end = 0.02
ddim_steps = 2
images = images.bin
H = 28
W = 28
C = 1
seed = 4242
tf32 = 0
save_every = {steps}
ckpt_dir = ckpt
"""


def _read_training_checkpoint(path):
    """src/checkpoint.c:92-136: magic 'CKTR', step, adam_t, then four lists (parameters, EMA shadows,
    Adam m, Adam v), each = count, per-tensor sizes, float payloads."""
    raw = Path(path).read_bytes()
    magic, step, adam_t = struct.unpack_from("<Iii", raw, 0)
    assert magic == 0x434B5452
    off, lists = 12, []
    for _ in range(4):
        (count,) = struct.unpack_from("<i", raw, off)
        sizes = struct.unpack_from(f"<{count}i", raw, off + 4)
        off += 4 + 4 * count
        total = sum(sizes)
        lists.append((sizes, np.frombuffer(raw, np.float32, total, off)))
        off += 4 * total
    assert off == len(raw)
    return step, adam_t, lists


def _train(exe, folder):
    folder.mkdir()
    rng = np.random.default_rng(0)
    img = np.where(rng.random((256, 28, 28)) < 0.8, -1.0, rng.uniform(-1, 1, (256, 28, 28))).astype(np.float32)
    img.tofile(folder / "images.bin")
    (folder / "ddpm.ini").write_text(INI.format(steps=STEPS))
    res = subprocess.run([str(exe), "ddpm.ini"], cwd=folder, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    loss = [float(ln.split()[3]) for ln in res.stdout.splitlines() if ln.startswith("step")]
    step, adam_t, lists = _read_training_checkpoint(folder / "ckpt" / f"step_{STEPS}.ckpt")
    assert step == STEPS and adam_t == STEPS
    return loss, lists


def _need(*exes):
    for e in exes:
        if not e.exists():
            pytest.skip(f"{e.name} not built (needs the reference sources at build time)")


def _worst(a, b):
    """Largest difference over the four lists, each relative to the list's largest magnitude."""
    return max(float(np.abs(x[1] - y[1]).max()) / max(float(np.abs(y[1]).max()), 1e-12) for x, y in zip(a, b))


def test_ddpm_trainer_fused_block_matches_plain_drop_in(tmp_path):
    """The reference's DDPM trainer on this library, with and without the replaced host modules: same
    parameter list layout, same first loss, parameters / shadows / moments equal to fp32 round-off."""
    _need(BIN / "ddpm_demo_b200", BIN / "ddpm_demo_b200_fused")
    loss_a, a = _train(BIN / "ddpm_demo_b200", tmp_path / "plain")
    loss_b, b = _train(BIN / "ddpm_demo_b200_fused", tmp_path / "fused")
    assert [x[0] for x in a] == [x[0] for x in b], "parameter list layout differs"
    assert len(a[0][0]) > 50 and sum(a[0][0]) > 500_000
    assert abs(loss_a[0] - loss_b[0]) <= 1e-5 * abs(loss_a[0])
    worst = _worst(a, b)
    print("ddpm: fused block vs plain drop-in, worst relative difference after", STEPS, "steps:", worst)
    assert worst <= 1e-4
    assert np.isfinite(a[0][1]).all() and np.isfinite(b[0][1]).all()


def test_ddpm_trainer_matches_reference_kernels_to_the_reference_own_spread(tmp_path):
    _need(BIN / "ddpm_demo_b200", REFBIN / "ddpm_demo_ref")
    loss_o, ours = _train(BIN / "ddpm_demo_b200", tmp_path / "ours")
    loss_o2, ours2 = _train(BIN / "ddpm_demo_b200", tmp_path / "ours2")
    refs = [_train(REFBIN / "ddpm_demo_ref", tmp_path / f"ref{i}") for i in range(5)]
    # this library is reproducible run to run (its only float atomics are in g_gain of the weight norm,
    # which the DDPM network does not use)
    self_spread = _worst(ours, ours2)
    assert self_spread <= 1e-5 and all(np.isfinite(x[1]).all() for x in ours)
    # the reference is not: the race in its GroupNorm kernels changes results from run to run and can leave
    # non-finite values in the state; only its finite runs can serve as a yardstick
    finite = [r for r in refs if all(np.isfinite(x[1]).all() for x in r[1]) and np.isfinite(r[0]).all()]
    dists = [_worst(ours, r[1]) for r in finite]
    spread = max([_worst(finite[i][1], finite[j][1]) for i in range(len(finite)) for j in range(i)] or [float("nan")])
    print(f"ddpm after {STEPS} fp32 steps: this library run-to-run {self_spread:.2e}; reference: {len(finite)} of "
          f"{len(refs)} runs finite, run-to-run {spread:.2e}; this library vs reference runs {[f'{d:.2e}' for d in dists]}; "
          f"first losses ours {loss_o[0]:.6f} reference {[round(r[0][0], 6) for r in refs]}")
    for r in finite:
        assert abs(loss_o[0] - r[0][0]) <= 1e-2 * abs(r[0][0])
    if len(finite) >= 2:
        assert max(dists) <= 2.0 * spread + 1e-4
    elif finite:
        assert max(dists) <= 5e-2


def test_ddpm_block_gradients_by_central_differences():
    """tests/host/ddpm_block_gradcheck.c: the replaced residual block (fused GroupNorm+SiLU, recomputed
    pre-activation) against central differences of L = <forward(x), g> for the input, the time embedding
    and every parameter tensor, three block shapes."""
    _need(BIN / "ddpm_block_gradcheck")
    res = subprocess.run([str(BIN / "ddpm_block_gradcheck")], capture_output=True, text=True, timeout=600)
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "0 failure(s)" in res.stdout and res.stdout.count("PASS") == 3 * 12 and "FAIL" not in res.stdout


def test_ddpm_dp_step_matches_reference_step():
    """csrc/host/ddpm_dp_train.c --check: the batched data-parallel step (one launch for the forward diffusion,
    one for the min-SNR-weighted loss gradient, pinned uploads) against the reference's own ddpm_loss_step on the
    same model from the same host and device random state: same loss, same gradients."""
    _need(BIN / "ddpm_dp_train")
    res = subprocess.run([str(BIN / "ddpm_dp_train"), "--check"], capture_output=True, text=True, timeout=600)
    print(res.stdout[-2000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "0 failure(s)" in res.stdout and res.stdout.count("PASS") == 2


def _dp_dump(tmp_path, name, extra, world=1):
    import os
    exe = BIN / "ddpm_dp_train"
    dump = tmp_path / f"{name}.bin"
    args = [str(exe), "--fp32", "--steps", "3", "--warmup", "2", "--batch", "16", "--dump", str(dump), *extra]
    if world == 1:
        res = subprocess.run(args, capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
        out = res.stdout
    else:
        procs = []
        for r in range(world):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), NCCL_NVLS_ENABLE="0")
            procs.append(subprocess.Popen(args + ["--id-file", str(tmp_path / f"{name}.id")], env=env,
                                          stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
        outs = [p.communicate(timeout=180) for p in procs]
        assert all(p.returncode == 0 for p in procs), outs
        out = outs[0][0]
    import json
    got = json.loads(next(ln for ln in out.splitlines() if ln.startswith("{")))["ddpm_dp_train"]
    return np.fromfile(dump, dtype=np.float32), got


def test_ddpm_dp_trainer_graph_and_sharded_optimizer_agree_with_eager(tmp_path):
    """Five fp32 steps: eager, replayed from a CUDA graph, and with the range-sharded optimizer (world = 1) end
    in the same parameters."""
    _need(BIN / "ddpm_dp_train")
    a, ga = _dp_dump(tmp_path, "eager", [])
    b, gb = _dp_dump(tmp_path, "graph", ["--graph"])
    c, gc = _dp_dump(tmp_path, "sharded", ["--sharded", "allgather"])
    assert a.size > 900_000 and ga["replicas_in_sync"] and gb["cuda_graph_nodes"] > 100
    assert np.isfinite(a).all() and np.isfinite(ga["last_loss"])
    assert np.array_equal(a, b)
    assert np.abs(a[1:] - c[1:]).max() <= 1e-6 * np.abs(a[1:]).max()


def test_ddpm_dp_trainer_two_ranks(tmp_path):
    """2 GPUs: replicas stay in sync with the all-reduce and with the sharded optimizer's peer stores, and both
    end in the same parameters up to the order of the gradient sums."""
    import torch
    _need(BIN / "ddpm_dp_train")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    a, ga = _dp_dump(tmp_path, "replicated", ["--graph"], world=2)
    b, gb = _dp_dump(tmp_path, "sharded", ["--graph", "--sharded", "peer"], world=2)
    assert ga["replicas_in_sync"] and gb["replicas_in_sync"] and ga["n_gpus"] == 2
    assert np.abs(a[1:] - b[1:]).max() <= 5e-5 * np.abs(a[1:]).max()
