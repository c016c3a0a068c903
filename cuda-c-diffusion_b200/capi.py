"""ctypes binding of libb200_layer_kernels.so (the C ABI in include/b200_layer_kernels.h).

Loading fails loudly when the library has not been built: there is no CPU or
PyTorch fallback behind these entry points.

Signature codes: p = device pointer, i = int, f = float, q = long long,
s = cudaStream_t, h = host pointer.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_NAME = "libb200_layer_kernels.so"
LIB_PATH = Path(__file__).resolve().parent / LIB_NAME

# name -> argument codes; every function returns void unless listed in RETURNS
SIGNATURES = {
    # part 1: the reference launcher set (src/nn.h:354-462)
    "launch_add_bias": "ppiis",
    "launch_activation_forward": "ppiis",
    "launch_activation_backward": "pppiis",
    "launch_softmax_xent": "ppppiis",
    "launch_bias_grad": "ppiis",
    "launch_sgd_step": "ppfis",
    "launch_adam_step": "ppppffffffis",
    "launch_weight_normalize": "piifs",
    "launch_weight_normalize_backward": "ppppiis",
    "launch_scale_by_scalar": "ppis",
    "launch_mp_sum": "pppfis",
    "launch_weighted_sum": "pppffis",
    "launch_mp_fourier": "ppppiis",
    "launch_modulate": "pppis",
    "launch_modulate_backward": "pppppis",
    "launch_sinusoidal": "ppiifs",
    "launch_embed_gather": "pppiiis",
    "launch_embed_scatter": "pppiiis",
    "launch_layernorm_forward": "ppppppiifs",
    "launch_layernorm_backward": "ppppppppiis",
    "launch_groupnorm_forward": "ppppppiiiifs",
    "launch_groupnorm_backward": "ppppppppiiiis",
    "launch_mp_cat": "pppfiiis",
    "launch_im2col": "ppiiiiiiiiis",
    "launch_col2im": "ppiiiiiiiiis",
    "launch_avg_pool_2x": "ppiiiis",
    "launch_avg_pool_2x_backward": "ppiiiis",
    "launch_nearest_upsample_2x": "ppiiiis",
    "launch_nearest_upsample_2x_backward": "ppiiiis",
    "launch_attn_softmax": "ppiis",
    "launch_attn_softmax_backward": "pppiis",
    "launch_permute_0213": "ppiiiis",
    "launch_spatial_modulate": "pppiiiis",
    "launch_spatial_modulate_backward": "pppppiiiis",
    "launch_spatial_add": "ppiiiis",
    "launch_spatial_reduce_sum": "ppiiis",
    "launch_channel_cat": "pppiiis",
    "launch_channel_split": "pppiiis",
    "launch_mp_channel_cat": "pppfiiis",
    "launch_mp_channel_split": "pppfiiis",
    "launch_mse_fwd_bwd": "ppppiis",
    "launch_clamp": "pffis",
    # part 2: additive fused entry points
    "launch_groupnorm_act_forward": "ppppppiiiifis",
    "launch_groupnorm_act_backward": "pppppppppiiiiis",
    "launch_pixel_norm_forward": "ppiifs",
    "launch_pixel_norm_backward": "pppiifs",
    "launch_mp_sum_backward": "pppfis",
    "launch_adam_ema_step": "pppppffffffffqs",
    "launch_adam_ema_step_multi": "hiffffffffs",
    "launch_weight_normalize_multi": "hifs",
    "launch_weight_normalize_backward_multi": "his",
    "b200_wn_batch_mode": "i",
    "b200_wn_forward_all": "s",
    "b200_wn_backward_flush": "s",
    "launch_axpby_rows": "pppppiis",
    "launch_col2im_assign": "ppiiiiiiiiis",
    "launch_film_act_forward": "pppiiiiis",
    "launch_film_act_backward": "pppppiiiiis",
    "launch_activation_backward_axpy": "ppppfiis",
    "launch_layernorm_backward_noalloc": "ppppppppiis",
    "launch_adam_ema_step_bcast": "ppppphffffffffqs",
    "launch_copy_multi": "his",
    # management
    "b200_set_error_mode": "i",
    "b200_error_count": "",
    "b200_last_error": "hi",
    "b200_clear_error": "",
    "b200_device_error_status": "",
    "b200_launch_count": "",
    "b200_launch_count_reset": "",
    "b200_groupnorm_path_count": "i",
    "b200_groupnorm_describe": "iiiiiihi",
    "b200_scratch_reserve": "sq",
    "b200_tune_set": "hi",
    "b200_tune_get": "hi",
    "b200_version": "",
}

RETURNS = {
    "launch_layernorm_backward_noalloc": ctypes.c_int,
    "b200_error_count": ctypes.c_int,
    "b200_wn_forward_all": ctypes.c_int,
    "b200_wn_backward_flush": ctypes.c_int,
    "b200_last_error": ctypes.c_int,
    "b200_device_error_status": ctypes.c_int,
    "b200_launch_count": ctypes.c_longlong,
    "b200_groupnorm_path_count": ctypes.c_longlong,
    "b200_groupnorm_describe": ctypes.c_int,
    "b200_scratch_reserve": ctypes.c_int,
    "b200_tune_get": ctypes.c_int,
    "b200_version": ctypes.c_char_p,
}

# the 42 launchers the reference declares (drop-in set)
REFERENCE_LAUNCHERS = [n for n in list(SIGNATURES)[:42]]

_CODES = {
    "p": ctypes.c_void_p,
    "h": ctypes.c_void_p,
    "s": ctypes.c_void_p,
    "i": ctypes.c_int,
    "f": ctypes.c_float,
    "q": ctypes.c_longlong,
}


class ParamUpdate(ctypes.Structure):
    """B200ParamUpdate of include/b200_layer_kernels.h."""
    _fields_ = [("p", ctypes.c_void_p), ("g", ctypes.c_void_p), ("m", ctypes.c_void_p),
                ("v", ctypes.c_void_p), ("shadow", ctypes.c_void_p), ("n", ctypes.c_int)]


class PeerDests(ctypes.Structure):
    """B200PeerDests of include/b200_layer_kernels.h."""
    _fields_ = [("dst", ctypes.c_void_p * 15), ("count", ctypes.c_int)]


class CopyItem(ctypes.Structure):
    """B200CopyItem of include/b200_layer_kernels.h."""
    _fields_ = [("dst", ctypes.c_void_p), ("src", ctypes.c_void_p), ("n", ctypes.c_int)]


class WeightDesc(ctypes.Structure):
    """B200WeightDesc of include/b200_layer_kernels.h."""
    _fields_ = [("W", ctypes.c_void_p), ("rows_in", ctypes.c_int), ("cols_out", ctypes.c_int)]


class WeightGradDesc(ctypes.Structure):
    """B200WeightGradDesc of include/b200_layer_kernels.h."""
    _fields_ = [("gW", ctypes.c_void_p), ("Wn", ctypes.c_void_p), ("gain", ctypes.c_void_p), ("g_gain", ctypes.c_void_p),
                ("rows_in", ctypes.c_int), ("cols_out", ctypes.c_int)]


def bind(lib: ctypes.CDLL, signatures=None) -> ctypes.CDLL:
    """Attach argtypes/restype for every declared symbol; raises if one is missing."""
    for name, codes in (signatures or SIGNATURES).items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise ImportError(f"{LIB_NAME} does not export {name}") from exc
        fn.argtypes = [_CODES[c] for c in codes]
        fn.restype = RETURNS.get(name)
    return lib


_lib = None


def load() -> ctypes.CDLL:
    """Load (once) and return the bound library.  No fallback: a missing build is an error."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python cuda-c-diffusion_b200/build.py` "
                "(there is no CPU fallback for these kernels)")
        _lib = bind(ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_LOCAL))
    return _lib
