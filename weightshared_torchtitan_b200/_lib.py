"""ctypes binding of libwsl.so (include/wsl.h). No torch types cross this boundary:
pointers are passed as integers, sizes as 64-bit ints, the stream as a raw handle.

There is no fallback: if the library is missing the first call raises.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libwsl.so")

WSL_BF16 = 0
WSL_F32 = 1
WSL_OK = 0
WSL_ERR_BAD_ARG = -1
WSL_ERR_ALIGN = -2
WSL_ERR_DEVICE = -3
WSL_ERR_CUDA = -4
WSL_ERR_TIMEOUT = -5
WSL_ERR_DRIVER = -6
WSL_ERR_TOO_LARGE = -7

# wsl_set_option / wsl_get_option keys
OPT_WAIT_LIMIT_MS = 1
OPT_STALL_PRODUCER = 2
OPT_PAIR_TILES = 3
OPT_ROW_STAGED = 4
OPT_RESERVED_SMS = 5
OPT_PROFILE_BITS = 6
OPT_MERGE_SIMT = 7
OPT_GRID_WAVES = 8
OPT_SPLIT_TAIL = 9
OPT_DEPENDENT_LAUNCH = 10

_vp = ctypes.c_void_p
_ll = ctypes.c_longlong
_i = ctypes.c_int
_f = ctypes.c_float
_vpp = ctypes.POINTER(ctypes.c_void_p)
_llp = ctypes.POINTER(ctypes.c_longlong)

# name -> (restype, argtypes); mirrors include/wsl.h one to one.
SIGNATURES = {
    "wsl_version": (_i, []),
    "wsl_status_string": (ctypes.c_char_p, [_i]),
    "wsl_launch_count": (ctypes.c_ulonglong, []),
    "wsl_poll_status": (_i, [ctypes.POINTER(_i)]),
    "wsl_reset_status": (_i, []),
    "wsl_set_option": (_i, [_i, _ll]),
    "wsl_get_option": (_ll, [_i]),
    "wsl_linear_fwd": (_i, [_vp, _ll, _vp, _vp, _ll, _ll, _ll, _ll, _i, _i, _vp]),
    "wsl_lora_prepass": (_i, [_vp, _ll, _vp, _vp, _ll, _ll, _ll, _ll, _f, _i, _vp]),
    "wsl_lora_linear_fwd": (_i, [_vp, _ll, _vp, _vp, _ll, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _i, _vp]),
    "wsl_lora_linear_fwd_group": (_i, [_i, _vp, _ll, _vpp, _vpp, _llp, _vpp, _vpp, _llp, _llp, _llp, _ll, _ll, _vp]),
    "wsl_lora_swiglu_supported": (_i, [_ll, _ll, _ll, _ll]),
    "wsl_lora_swiglu_fwd": (_i, [_vp, _ll, _vp, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _vp]),
    "wsl_swiglu_bwd_in_dx_supported": (_i, [_ll, _ll, _ll, _ll]),
    "wsl_lora_linear_bwd_dx_swiglu": (_i, [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _vp]),
    "wsl_lora_bwd_prepass": (_i, [_vp, _ll, _vp, _vp, _ll, _ll, _ll, _ll, _f, _i, _vp]),
    "wsl_lora_linear_bwd_dx": (_i, [_i, _vpp, _llp, _vpp, _llp, _vpp, _vpp, _llp, _llp, _vp, _ll, _ll, _ll, _i, _vp]),
    "wsl_lora_linear_bwd_dw": (_i, [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _ll, _ll, _ll, _ll,
                                    _vp, ctypes.c_ulonglong, _i, _vp]),
    "wsl_lora_linear_bwd_dw_noalloc": (_i, [_vp, _ll, _vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _vp]),
    "wsl_lora_linear_bwd_dw_group": (_i, [_i, _vpp, _llp, _vpp, _llp, _vp, _ll, _vpp, _llp, _vpp, _vpp, _vpp,
                                          _llp, _llp, _ll, _ll, _vp, ctypes.c_ulonglong, _vp]),
    "wsl_bwd_dw_group_workspace_bytes": (ctypes.c_ulonglong, [_i, _llp, _llp, _ll, _ll]),
    "wsl_lora_merge_weight": (_i, [_i, _vpp, _vpp, _vpp, _vpp, _llp, _ll, _ll, _f, _vp]),
    "wsl_adapter_grads_workspace_bytes": (ctypes.c_ulonglong, [_i, _llp, _llp, _llp]),
    "wsl_bwd_dw_layer_group": (_i, [_i, _vpp, _llp, _vp, _ll, _vpp, _vpp, _llp, _ll, _ll, _vp,
                                    ctypes.c_ulonglong, _vp]),
    "wsl_lora_adapter_grads_from_dw": (_i, [_i, _vpp, _vpp, _vpp, _vpp, _vpp, _llp, _llp, _llp, _f, _vp,
                                            ctypes.c_ulonglong, _vp]),
    "wsl_bwd_dw_workspace_bytes": (ctypes.c_ulonglong, [_ll, _ll, _ll, _ll, _i, _i, _i]),
    "wsl_ce_fwd_bwd": (_i, [_vp, _ll, _vp, _vp, _ll, _ll, _f, _vp, _i, _vp]),
    "wsl_swiglu_fwd": (_i, [_vp, _vp, _vp, _ll, _i, _vp]),
    "wsl_swiglu_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _ll, _i, _vp]),
    "wsl_rmsnorm_fwd": (_i, [_vp, _ll, _vp, _vp, _ll, _vp, _ll, _ll, _f, _vp, _vp, _ll, _ll, _i, _vp]),
    "wsl_rmsnorm_bwd": (_i, [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _ll, _vp, _vp, _ll, _ll, _i, _vp]),
    "wsl_add_rmsnorm_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _f, _i, _vp]),
    "wsl_grad_sumsq_partials": (_i, [_vp, _ll, _vp, _vp]),
    "wsl_adamw_flat_step": (_i, [_vp, _vp, _vp, _vp, _vp, _ll, _f, _f, _f, _f, _f, _f, _f, _vp, _i, _f, _vp]),
    "wsl_add_rmsnorm_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _vp]),
    "wsl_embed_fwd": (_i, [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _vp]),
    "wsl_embed_bwd_dproj": (_i, [_vp, _vp, _ll, _vp, _vp, _ll, _ll, _ll, _ll, _vp, ctypes.c_ulonglong, _vp]),
    "wsl_embed_gather": (_i, [_vp, _vp, _vp, _ll, _ll, _ll, _i, _vp]),
    "wsl_embed_scatter_add": (_i, [_vp, _vp, _vp, _ll, _ll, _ll, _i, _vp]),
}

_LIB = None


class WslError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: wsl status {status}: {status_string(status)}")


def lib() -> ctypes.CDLL:
    """Load libwsl.so once. Raises if it has not been built (no CPU fallback exists)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with "
                "`python -m weightshared_torchtitan_b200.build` (needs nvcc); "
                "this package has no fallback path"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def status_string(status: int) -> str:
    return lib().wsl_status_string(status).decode()


def check(status: int, where: str) -> None:
    if status != WSL_OK:
        raise WslError(status, where)


def poll_status():
    """(status, [4 words]) of the current device; see wsl_poll_status in include/wsl.h."""
    words = (ctypes.c_int * 4)()
    st = lib().wsl_poll_status(words)
    return st, list(words)


def launch_count() -> int:
    return int(lib().wsl_launch_count())


def set_option(option: int, value: int) -> None:
    """Process-wide run-time option of the library (see wsl_set_option in include/wsl.h)."""
    check(lib().wsl_set_option(option, int(value)), "wsl_set_option")


def get_option(option: int) -> int:
    return int(lib().wsl_get_option(option))
