"""CPU: the partition arithmetic of the range-sharded optimizer (csrc/host/b200_shard_plan.c), built with gcc
alone and run here -- ranges tile the padded vector, tensor layout, ownership of every element, and the
failure forms (bad rank, empty world, negative size, a peer that reports another model / shard / world)."""
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_shard_plan_host_check(tmp_path):
    exe = tmp_path / "shard_plan_check"
    subprocess.run(["gcc", "-O2", "-std=c11", "-Wall", "-Werror", f"-I{ROOT / 'include'}",
                    str(ROOT / "tests" / "host" / "shard_plan_check.c"),
                    str(ROOT / "cuda-c-diffusion_b200" / "csrc" / "host" / "b200_shard_plan.c"), "-o", str(exe)],
                   check=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0 and "0 failure(s)" in res.stdout, res.stdout[-2000:]
