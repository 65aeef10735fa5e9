"""ctypes binding of libmta_b200.so, the C-ABI CUDA library (see include/mta_b200.h).

There is no fallback: if the shared library has not been built, importing the ops raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmta_b200.so")

MTA_F32, MTA_BF16, MTA_F16 = 0, 1, 2
DTYPE_CODE = {torch.float32: MTA_F32, torch.bfloat16: MTA_BF16, torch.float16: MTA_F16}

_lib: Optional[ctypes.CDLL] = None

# name -> (restype, argtypes); kept in one table so a test can check it against the header.
_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
SIGNATURES = {
    "mta_abi_version": (_i, []),
    "mta_last_error": (ctypes.c_char_p, []),
    "mta_launch_count": (ctypes.c_long, []),
    "mta_reset_launch_count": (None, []),
    "mta_set_variant": (_i, [ctypes.c_char_p, _i]),
    "mta_inject_wait_timeout": (_i, [_vp]),
    "mta_device_status": (_i, [_vp]),
    "mta_conv2d_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "mta_head_linear_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp]),
    "mta_softmax_fwd": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "mta_head_linear_softmax_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "mta_conv2d_bwd_input": (_i, [_vp, _vp, _vp] + [_i] * 9 + [_vp]),
    "mta_conv2d_bwd_weight_workspace_bytes": (_sz, [_i] * 6),
    "mta_conv2d_bwd_weight": (_i, [_vp, _vp, _vp, _vp, _sz] + [_i] * 8 + [_vp]),
    "mta_head_linear_bwd_input": (_i, [_vp, _vp, _vp] + [_i] * 7 + [_vp]),
    "mta_head_linear_bwd_weight_workspace_bytes": (_sz, [_i]),
    "mta_head_linear_bwd_weight": (_i, [_vp, _vp, _vp, _vp, _sz] + [_i] * 6 + [_vp]),
    "mta_qk_scores_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _i, _vp]),
    "mta_pv_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "mta_conv_attn_workspace_bytes": (_sz, [_i] * 9),
    "mta_conv_attn_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _vp]),
    "mta_static_scratch_bytes": (_sz, []),
    "mta_static_scratch_prepare": (_i, []),
    "mta_conv_attn_fwd_static": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _vp]),
    "mta_workspace_bytes": (_sz, [_i] * 11),
    "mta_fused_fwd": (_i, [_vp] * 9 + [_sz] + [_i] * 13 + [_vp]),
    "mta_fused_fwd_dropout": (_i, [_vp] * 9 + [_sz] + [_i] * 13 + [_f, ctypes.c_ulonglong, _vp]),
    "mta_fused_fwd_host": (_i, [_vp] * 8 + [_i] * 12),
    "mta_host_pipeline_release": (_i, []),
    "mta_set_stage_trace": (_i, [_i]),
    "mta_stage_times_ms": (_i, [_vp, _vp, _i]),
}


class MTALibraryError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it was not built: there is no CPU or PyTorch fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MTALibraryError(
                f"{LIB_PATH} is missing: build it with `python -m multitokenatention_triton_b200.build` "
                "(nvcc, sm_100a). This package has no fallback path.")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().mta_last_error().decode("utf-8", "replace")
        kind = {1: "invalid argument", 2: "CUDA error", 3: "wrong architecture", 4: "device-side timeout"}.get(rc, "error")
        raise MTALibraryError(f"{what}: {kind} (status {rc}): {msg}")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise MTALibraryError(f"unsupported dtype {t.dtype}: expected float32, bfloat16 or float16") from None


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def device_status(device=None) -> None:
    """Synchronises the current stream and raises if a device-side bounded wait gave up."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        check(lib().mta_device_status(stream_ptr(dev)), "mta_device_status")


def set_variant(key: str, value: int) -> None:
    check(lib().mta_set_variant(key.encode(), int(value)), f"set_variant({key})")


def launch_count() -> int:
    return int(lib().mta_launch_count())


def reset_launch_count() -> None:
    lib().mta_reset_launch_count()


def set_stage_trace(on: bool) -> None:
    """Switches the per-stage CUDA-event tracing of mta_fused_fwd on or off for the calling thread."""
    check(lib().mta_set_stage_trace(int(bool(on))), "mta_set_stage_trace")


def stage_times_ms():
    """[(stage name, device milliseconds)] of the latest traced mta_fused_fwd (waits for it to finish)."""
    ms = (ctypes.c_float * 8)()
    names = (ctypes.c_char_p * 8)()
    n = lib().mta_stage_times_ms(ms, names, 8)
    if n < 0:
        raise MTALibraryError("mta_stage_times_ms: CUDA error while reading the stage events")
    return [(names[i].decode(), float(ms[i])) for i in range(n)]
