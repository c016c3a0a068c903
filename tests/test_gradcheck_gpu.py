"""Runs the reference's own finite-difference test (tests/gradcheck.c, unmodified,
with its unmodified host modules) linked against this library's kernels.  The
binaries are built by cuda-c-diffusion_b200/csrc/host/Makefile where the reference sources are available."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "cuda-c-diffusion_b200" / "build" / "bin"  # built by cuda-c-diffusion_b200/csrc/host/Makefile


def _run(exe):
    if not exe.exists():
        pytest.skip(f"{exe.name} not built (needs the reference sources at build time)")
    return subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)


def test_reference_gradcheck_passes_with_our_kernels():
    res = _run(BIN / "gradcheck_b200")
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "ALL GRADIENTS OK" in res.stdout
    assert res.stdout.count("[PASS]") == 15


def test_c_host_modules_of_fused_entry_points():
    """csrc/host/b200_fused_modules.c (Module vtable + public optimizer/EMA API of the reference)
    against the reference's own host modules and central differences; see tests/host/."""
    res = _run(BIN / "fused_modules_check")
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "0 failure(s)" in res.stdout
    assert res.stdout.count("PASS") == 25 and "FAIL" not in res.stdout


def test_edm_dp_step_matches_reference_step():
    """csrc/host/edm_dp_train.c --check: the batched data-parallel step against the reference's own
    edm_loss_step + optimizer_step + ema_update from identical state (fp32 GEMMs, two steps)."""
    res = subprocess.run([str(BIN / "edm_dp_train"), "--check"], capture_output=True, text=True,
                         timeout=600) if (BIN / "edm_dp_train").exists() else None
    if res is None:
        pytest.skip("edm_dp_train not built (needs the reference sources at build time)")
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "0 failure(s)" in res.stdout and res.stdout.count("PASS") == 9


def test_edm_dp_two_ranks_stay_in_sync(tmp_path):
    """Two trainer processes, one per GPU, NCCL gradient all-reduce: replicas must hold identical parameters
    after the run, eager and with the CUDA graph."""
    import json
    import os
    import torch
    exe = BIN / "edm_dp_train"
    if not exe.exists():
        pytest.skip("edm_dp_train not built (needs the reference sources at build time)")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    for extra in ([], ["--graph"]):
        id_file = tmp_path / ("id" + "_".join(extra))
        procs = []
        for r in range(2):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), NCCL_NVLS_ENABLE="0")
            procs.append(subprocess.Popen([str(exe), "--batch", "16", "--steps", "4", "--warmup", "3", "--id-file",
                                           str(id_file)] + extra, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                          text=True))
        try:
            outs = [p.communicate(timeout=120) for p in procs]
        except subprocess.TimeoutExpired:
            for p in procs:
                p.kill()
            pytest.fail(f"trainer ranks did not finish within 120 s ({extra})")
        assert all(p.returncode == 0 for p in procs), outs
        line = next(ln for ln in outs[0][0].splitlines() if ln.startswith("{"))
        got = json.loads(line)["edm_dp_train"]
        assert got["replicas_in_sync"] is True and got["n_gpus"] == 2 and got["b200_device_error"] == 0


def test_reference_gradcheck_passes_with_replaced_conv2d_host_module():
    """The reference's gradcheck with its conv2d.c replaced at link time by csrc/host/b200_conv2d.c."""
    res = _run(BIN / "gradcheck_b200_fastconv")
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "ALL GRADIENTS OK" in res.stdout
    assert res.stdout.count("[PASS]") == 15


def test_replaced_conv2d_trains_to_the_same_parameters(tmp_path):
    """Five fp32 training steps with the reference's conv2d host module and with the replacement
    (gain as GEMM alpha, column buffer reused, 1x1 as plain GEMM) from the same seed: same loss and parameters."""
    import numpy as np
    outs = {}
    for name in ("edm_dp_train", "edm_dp_train_fastconv"):
        exe = BIN / name
        if not exe.exists():
            pytest.skip(f"{name} not built (needs the reference sources at build time)")
        dump = tmp_path / (name + ".bin")
        res = subprocess.run([str(exe), "--fp32", "--steps", "3", "--warmup", "2", "--batch", "16", "--dump", str(dump)],
                             capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
        outs[name] = np.fromfile(dump, dtype=np.float32)
    a, b = outs["edm_dp_train"], outs["edm_dp_train_fastconv"]
    assert a.size == b.size and a.size > 1_000_000
    assert abs(a[0] - b[0]) <= 1e-5 * abs(a[0])                       # loss of the last step
    assert np.abs(a[1:] - b[1:]).max() <= 1e-5 * np.abs(a[1:]).max()  # every parameter


def test_edm_dp_checkpoint_round_trip(tmp_path):
    """--save writes the reference's training checkpoint after the run; --resume restores parameters
    (and optimizer/EMA state) exactly and training continues from there."""
    import json
    import numpy as np
    exe = BIN / "edm_dp_train_fastconv"
    if not exe.exists():
        pytest.skip("edm_dp_train_fastconv not built (needs the reference sources at build time)")
    ck, d_a, d_b, d_c = (str(tmp_path / n) for n in ("state.ckpt", "a.bin", "b.bin", "c.bin"))
    run = lambda *a: subprocess.run([str(exe), "--fp32", "--batch", "8", *a], capture_output=True, text=True, timeout=300)
    res = run("--warmup", "2", "--steps", "2", "--save", ck, "--dump", d_a)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    res = run("--resume", ck, "--warmup", "0", "--steps", "0", "--dump", d_b)  # load and dump, no training
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    a, b = np.fromfile(d_a, dtype=np.float32), np.fromfile(d_b, dtype=np.float32)
    assert np.array_equal(a[1:], b[1:])
    res = run("--resume", ck, "--warmup", "2", "--steps", "2", "--dump", d_c)  # continue for four more steps
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    got = json.loads(next(ln for ln in res.stdout.splitlines() if ln.startswith("{")))["edm_dp_train"]
    c = np.fromfile(d_c, dtype=np.float32)
    assert np.isfinite(c).all() and not np.array_equal(c[1:], a[1:]) and np.isfinite(got["last_loss"])


def test_edm_dp_missing_peer_ends_with_an_error_not_a_hang(tmp_path):
    """Failure injected on the host: rank 1 of a world of two starts alone, so the NCCL id never appears.
    The rank must give up after its bounded wait with a clear message; nothing has touched the device."""
    import os
    import time
    exe = BIN / "edm_dp_train"
    if not exe.exists():
        pytest.skip("edm_dp_train not built (needs the reference sources at build time)")
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="0", EDM_DP_ID_WAIT_S="1.5")
    t0 = time.time()
    res = subprocess.run([str(exe), "--batch", "8", "--steps", "1", "--warmup", "0", "--id-file", str(tmp_path / "never")],
                         env=env, capture_output=True, text=True, timeout=120)
    assert res.returncode != 0
    assert "did not publish the NCCL id" in res.stderr
    assert time.time() - t0 < 60
