"""B200 (sm_100a) layer kernels behind the reference's `launch_*` C ABI.

The product is `libb200_layer_kernels.so` (sources in `csrc/`, header in
`include/b200_layer_kernels.h`).  This package only builds it (`build.py`),
binds it (`capi.py`) and offers tensor-level wrappers (`ops.py`) and the torch.distributed
form of the multi-GPU partitioning (`sharding.py`).  The host side proper is C: the reference's own
modules linked against the library, plus `csrc/host/` (fused modules, replaced residual blocks and
conv2d, data-parallel trainer, range-sharded optimizer).

The directory name contains a hyphen, so import it with
`importlib.import_module("cuda-c-diffusion_b200")`.
"""
from . import capi  # noqa: F401

__all__ = ["capi", "build", "ops", "sharding"]
