"""Generates tests/golden/reference_kernels.npz and tests/golden/reference_plain_launchers.npz:
outputs of the reference's OWN CUDA kernels (src/kernels.cu compiled unmodified for sm_100a into
oracle/_ref/, see oracle/Makefile) on the seeded inputs of tests/cases.py (the fused layer
kernels) and tests/plain_cases.py (the launchers either side of them).  Run on a machine with a GPU:

    python tests/golden/make_golden.py [output folder]

The reference has no CPU path and ships no golden vectors, so these files are what pins the CPU
oracle to the reference when no GPU is present (tests/test_oracle_golden.py).  Embedding cases use
the build without --use_fast_math; every other case uses the reference's own flags.
"""
import ctypes
import importlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
import cases  # noqa: E402
import plain_cases  # noqa: E402


def main():
    folder = Path(sys.argv[1]) if len(sys.argv) > 1 else ROOT / "tests" / "golden"
    out = folder / "reference_kernels.npz"
    capi = importlib.import_module("cuda-c-diffusion_b200.capi")
    sigs = {k: capi.SIGNATURES[k] for k in capi.REFERENCE_LAUNCHERS}
    fast = capi.bind(ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libref_kernels.so"), mode=ctypes.RTLD_LOCAL), sigs)
    precise = capi.bind(ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libref_kernels_precise.so"),
                                    mode=ctypes.RTLD_LOCAL), sigs)
    blob = {}
    for name, op, p in cases.CASES:
        inp = cases.make_inputs(op, p, seed=cases.seed_of(name))
        lib = precise if op in ("mp_fourier", "sinusoidal") else fast
        res = cases.gpu_run(lib, op, p, inp, fused=False)
        for k, v in res.items():
            blob[f"{name}/{k}"] = np.asarray(v, np.float32)
        # a fingerprint of the inputs guards against a drifting generator
        flat = np.concatenate([np.ravel(np.concatenate(v) if isinstance(v, list) else v).astype(np.float64)
                               for v in inp.values()])
        blob[f"{name}/__input_sum"] = np.array([flat.sum(), np.abs(flat).sum()])
    out.parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(out, **blob)
    print("wrote", out, sum(v.nbytes for v in blob.values()), "bytes raw")

    blob = {}
    for name, fn, args, _tol in plain_cases.PLAIN_CASES:
        for k, v in plain_cases.run_gpu(fast, name, fn, args).items():
            blob[f"{name}/{k}"] = v
        arrays, _ = plain_cases.materialise(name, args)
        flat = np.concatenate([np.ravel(v).astype(np.float64) for v in arrays.values()])
        blob[f"{name}/__input_sum"] = np.array([flat.sum(), np.abs(flat).sum()])
    out = folder / "reference_plain_launchers.npz"
    np.savez_compressed(out, **blob)
    print("wrote", out, sum(v.nbytes for v in blob.values()), "bytes raw")


if __name__ == "__main__":
    main()
