"""B200 (sm_100a) layer kernels behind the reference's `launch_*` C ABI.

The product is `libb200_layer_kernels.so` (sources in `csrc/`, header in
`include/b200_layer_kernels.h`).  This package only builds it (`build.py`),
binds it (`capi.py`) and offers tensor-level wrappers (`ops.py`), the host-side
mirror of the reference's Module interface (`modules.py`) and the multi-GPU
sharding helpers (`sharding.py`).

The directory name contains a hyphen, so import it with
`importlib.import_module("cuda-c-diffusion_b200")`.
"""
from . import capi  # noqa: F401

__all__ = ["capi", "build", "ops", "modules", "sharding"]
