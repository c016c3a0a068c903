"""GPU: the launchers either side of the fused layer kernels (tests/plain_cases.py), three ways.

* the CPU oracle against the reference's own kernels.cu built for sm_100a -- this is what pins
  that part of oracle/layer_oracle.c to reference src/kernels.cu:95-161 and :750-1313;
* this library against the reference's kernels (A/B);
* this library against the oracle.
"""
import pytest

import plain_cases as pc

pytestmark = pytest.mark.gpu

IDS = [c[0] for c in pc.PLAIN_CASES]


@pytest.mark.parametrize("name,fn,args,tol", pc.PLAIN_CASES, ids=IDS)
def test_oracle_agrees_with_reference_kernels(orc, ref_lib, name, fn, args, tol):
    pc.compare(pc.run_oracle(orc, name, fn, args), pc.run_gpu(ref_lib, name, fn, args), tol, "oracle/" + name)


@pytest.mark.parametrize("name,fn,args,tol", pc.PLAIN_CASES, ids=IDS)
def test_matches_reference_kernels(lib, ref_lib, name, fn, args, tol):
    pc.compare(pc.run_gpu(lib, name, fn, args), pc.run_gpu(ref_lib, name, fn, args), tol, name)


@pytest.mark.parametrize("name,fn,args,tol", pc.PLAIN_CASES, ids=IDS)
def test_matches_oracle(lib, orc, name, fn, args, tol):
    pc.compare(pc.run_gpu(lib, name, fn, args), pc.run_oracle(orc, name, fn, args), tol, name)
