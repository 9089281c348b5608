"""ctypes binding of libunica_b200.so, the C-ABI library declared in include/unica_b200.h.

The reference drives its kernels through the CUDA driver API from ctypes (unica/cuda.py: cubin -> cuModuleLoadData ->
cuLaunchKernel on torch's stream).  Here the same role is played by host entry points of one shared library, loaded
once per process; launches still go on torch's current stream of the current device.  There is no fallback: if the
library is missing and cannot be built, or an entry point fails, a RuntimeError says why (as unica/cuda.py:34-38 does
for driver errors).
"""

from __future__ import annotations

import ctypes
import functools
from pathlib import Path

HERE = Path(__file__).resolve().parent
import os  # noqa: E402

# UNICA_B200_LIB: another build of the same library (e.g. a -DUNICA_TRACE build from unicaattention_b200.build)
LIB_PATH = Path(os.environ["UNICA_B200_LIB"]) if "UNICA_B200_LIB" in os.environ else HERE / "libunica_b200.so"

ERR_ARGUMENT, ERR_CUDA, ERR_DEVICE, ERR_KERNEL = 1, 2, 3, 4
V_CHANNEL, V_TOKEN, V_OUTLIERS = 0, 1, 2


class TokenLayout(ctypes.Structure):
    """include/unica_b200.h unica_token_layout: strides in elements of a [batch, heads, tokens, 128] tensor, and its
    heads (the reference's TokenLayout, unica/__init__.py:92-100); dtype 0: bfloat16, 1: float16."""

    _fields_ = [("batch", ctypes.c_longlong), ("head", ctypes.c_longlong), ("token", ctypes.c_longlong),
                ("heads", ctypes.c_int), ("dtype", ctypes.c_int)]


_P, _I, _F, _LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
SIGNATURES = {
    # name: argument types (every entry point returns int)
    "unica_b200_version": [],
    "unica_b200_channel_stats": [_P, TokenLayout, _I, _I, _I, _P, _P, _P, _P, _P],
    "unica_b200_channel_stats_static": [_P, TokenLayout, _I, _I, _I, _P, _P, _P, _P],
    "unica_b200_quantize_int8": [_P, TokenLayout, _P, _I, _I, _I, _I, _P, _P, _P],
    "unica_b200_quantize_v_int8": [_P, TokenLayout, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P],
    "unica_b200_quantize_q_int8_stream": [_P, TokenLayout, _I, _I, _I, _P, _P, _P],
    "unica_b200_quantize_k_int8_fused": [_P, TokenLayout, _I, _I, _I, _P, ctypes.c_size_t, _P, _P, _P, _P, _P],
    "unica_b200_quantize_v_int8_fused": [_P, TokenLayout, _I, _I, _P, ctypes.c_size_t, _P, _P, _P, _P],
    "unica_b200_attention_int8": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _P, TokenLayout, _I, _I, _I, _F, _P, _P],
    "unica_b200_attention_int8_peers": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _P, _P, _I, TokenLayout, _I, _I, _I, _F, _P, _P],
    "unica_b200_attention_fp4_peers": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _I, TokenLayout, _I, _I, _I, _F, _P, _P],
    "unica_b200_channel_stats_masked": [_P, TokenLayout, _P, _I, _I, _P, _P, _P, _P, _P],
    "unica_b200_selftest_mma_i8": [_P, _P, _I, _I, _I, _I, _P, _P],
    "unica_b200_attention_fp4": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P, TokenLayout, _I, _I, _I, _F, _P, _P],
    "unica_b200_attention_fp4_codes": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P, TokenLayout, _I, _I, _I, _F, _P, _P, _P],
    "unica_b200_selftest_mma_nvf4": [_P, _P, _P, _P, _I, _I, _I, _P, _P],
    "unica_b200_peak": [_I, _I, _I, _I, _P, _P],
    "unica_b200_nvfp4_outer": [_P, _P, _P, _I, _I, _P, _P],
    "unica_b200_quantize_fp4_rows": [_P, TokenLayout, _P, _I, _P, _I, _I, _I, _I, _P, _P, _P],
    "unica_b200_quantize_v_fp4": [_P, TokenLayout, _P, _P, _I, _I, _P, _P, _P, _P],
    "unica_b200_smooth_bias": [_P, TokenLayout, _P, _P, _I, _I, _I, _F, _P, _P, _P],
    "unica_b200_channel_stats_rope": [_P, TokenLayout, _P, _LL, _I, _I, _I, _P, _P, _P, _P, _P],
    "unica_b200_quantize_int8_rope": [_P, TokenLayout, _P, _P, _LL, _I, _I, _I, _I, _P, _P, _P],
    "unica_b200_quantize_fp4_rows_rope": [_P, TokenLayout, _P, _I, _P, _LL, _P, _I, _I, _I, _I, _P, _P, _P],
    "unica_b200_smooth_bias_rope": [_P, TokenLayout, _P, _P, _P, _LL, _I, _I, _I, _F, _P, _P, _P],
}


@functools.cache
def library() -> ctypes.CDLL:
    """The loaded library.  Built in-tree with nvcc on first use when the source tree is there and the file is not."""
    if not LIB_PATH.exists():
        if (HERE / "csrc").exists():
            from unicaattention_b200.build import build

            build()
        else:
            raise RuntimeError(f"{LIB_PATH.name} is missing and there is no csrc/ to build it from")
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.unica_b200_last_error.restype = ctypes.c_char_p
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library is older than this binding
        fn.argtypes, fn.restype = argtypes, ctypes.c_int
    return lib


def last_error() -> str:
    message = library().unica_b200_last_error()
    return message.decode() if message else ""


def ptr(tensor) -> ctypes.c_void_p:
    """A tensor's device pointer, or NULL for None."""
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


def stream() -> ctypes.c_void_p:
    import torch

    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# kernels an entry point launches when it succeeds (the statistics passes: partial sums, then their reduction)
KERNELS_PER_CALL = {"unica_b200_channel_stats": 2, "unica_b200_channel_stats_rope": 2, "unica_b200_channel_stats_masked": 2,
                    "unica_b200_channel_stats_static": 2, "unica_b200_version": 0}
launches = 0  # kernels of this library launched by this process so far (benchmarks report differences of it)


def call(name: str, *args) -> None:
    """Run an entry point; ValueError for arguments it does not take, RuntimeError for everything else."""
    global launches
    code = getattr(library(), name)(*args)
    if code == 0:
        launches += KERNELS_PER_CALL.get(name, 1)
        return
    message = f"{name}: {last_error()}"
    raise ValueError(message) if code == ERR_ARGUMENT else RuntimeError(message)
