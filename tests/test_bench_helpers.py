"""CPU checks of bench.py's host logic: byte accounting, the trainer config writer, the roofline denominator,
and that the product arm refuses to run without a GPU (no CPU fallback)."""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_step_bytes_are_the_sum_of_the_kernels_algorithmic_bytes():
    b = _bench()
    assert sum(b.KERNEL_BYTES.values()) == b.STEP_BYTES
    n = b.B * b.HW * b.C
    assert b.KERNEL_BYTES["gn_silu_fwd"] == 2 * n * 4 and b.KERNEL_BYTES["gn_silu_bwd"] == 3 * n * 4
    assert set(b.NCU_TRAFFIC) <= set(b.KERNEL_BYTES)
    for k, traffic in b.NCU_TRAFFIC.items():  # measured DRAM traffic never exceeds the algorithmic bytes by much
        assert traffic <= 1.05 * b.KERNEL_BYTES[k]


def test_edm_config_writer(tmp_path):
    b = _bench()
    ini = b.write_edm_config(str(tmp_path), 256, 7)
    text = Path(ini).read_text()
    assert "train_steps = 7" in text and "batch_size = 256" in text and "channels = 64,128,128" in text
    img = np.fromfile(tmp_path / "images.bin", dtype=np.float32)
    assert img.size == 4096 * 28 * 28
    frac_background = float((img == -1.0).mean())
    assert 0.78 < frac_background < 0.82 and img.min() >= -1.0 and img.max() <= 1.0


def test_roofline_denominator_comes_from_the_measured_peaks_file():
    b = _bench()
    peak, src = b.measured_peak()
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        assert peak == float(json.loads(f.read_text())["hbm_gbs"]) and src.startswith("measured")
    else:
        assert peak == 6650.0 and src.startswith("fallback")


def test_product_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return  # this check is for the CPU box
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "1"], capture_output=True, text=True, timeout=300)
    assert res.returncode != 0 and "no CPU fallback" in (res.stderr + res.stdout)
