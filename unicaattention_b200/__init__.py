"""unicaattention_b200: UnicaAttention's forward quantized attention, rebuilt for the B200 (sm_100a).

    import unicaattention_b200 as unica
    out = unica.attention(q, k, v, **unica.PRESETS["per_channel"])   # [batch, heads, tokens, 128] bf16

The call surface is the reference's (unica/__init__.py): `attention`, `kernel_inputs`, `PRESETS`, the quantizer
functions, `TokenLayout`, the head-split planner, `compatibility`.  Underneath, every device step is an entry point of
libunica_b200.so (include/unica_b200.h): hand-written sm_100a kernels, tcgen05 tensor cores with accumulators in
tensor memory, K/V tiles staged by bulk TMA copies.  There is no CPU path and no other backend: without the library
or a B200 the calls raise.

What differs from the reference, on purpose: the packed operand layouts the quantizers return are this library's
(the shared-memory images of the tcgen05 operands, see include/unica_b200.h), not the sm_120 fragment layouts; the
`decode_*` helpers turn them back into plain [batch, heads, tokens, 128] codes for comparisons.  Build settings that
only steered the sm_120 kernels (WARPS_PER_BLOCK, PRODUCER, WAVE_DISPATCH) are accepted and have no effect.
"""

from __future__ import annotations

import ctypes
import functools
import math
import os
import time
import warnings
import weakref
from typing import Sequence

import torch

from unicaattention_b200 import lib
from unicaattention_b200.check import OK, UNSUPPORTED, UNTESTED, Compatibility, compatibility, machine  # noqa: F401
from unicaattention_b200.lib import TokenLayout

HEAD_DIM = 128
Q_SCALE_BLOCK = 128  # queries per Q scale = rows of one tcgen05.mma
K_SCALE_BLOCK = 64  # keys per K scale = keys per softmax tile (part of the numerics contract)
KEYS_PER_TILE = 64
V8_PAD_KEYS = 64  # V8 is padded to whole tiles
FP4_TILE = 64
STATS_TOKENS = 256
ROPE_PAIRS = HEAD_DIM // 2
MAX_OUTLIERS = 8  # outlier keys per head the accurate kernel adds back
LOG2E = 1.4426950408889634

# The two production modes, under the reference's kernel names (unica/__init__.py:34-40, 88-89).
KERNELS = ("attention_int8pv_tma", "attention_fp4")
QUANTIZED = set(KERNELS)
LAYOUT_KERNELS = set(KERNELS)  # both read q, k, v and write the output in the caller's layout
DEFAULT_KERNEL = "attention_int8pv_tma"
# Settings a call may pass (the reference's TILE).  The first three select numerics; the others steered the sm_120
# kernels' shape and are accepted for drop-in compatibility only.
TILE = {"V_TOKEN": 0, "V_OUTLIERS": 0, "SMOOTH_Q": 0, "KEYS_PER_TILE": 64, "WARPS_PER_BLOCK": 4, "PRODUCER": 0,
        "WAVE_DISPATCH": 0}
PRESETS = {"per_token": dict(V_TOKEN=1, WAVE_DISPATCH=1), "per_channel": dict(PRODUCER=1, WAVE_DISPATCH=1),
           "outliers": dict(V_OUTLIERS=8), "fast": dict(kernel="attention_fp4", SMOOTH_Q=512)}

VRAM_RESERVE: int | None = (int(os.environ["UNICA_VRAM_RESERVE_MB"]) * 2**20
                             if "UNICA_VRAM_RESERVE_MB" in os.environ else None)
LOG_VRAM = os.environ.get("UNICA_LOG_VRAM") == "1"
SMALL_CALL_FRACTION = 4


def warn_if_untested() -> None:
    """Says once, as the reference does on import, when this machine is not the measured combination."""
    status = compatibility()
    if status.status != OK:
        warnings.warn(str(status), stacklevel=2)


if os.environ.get("UNICA_QUIET") != "1" and torch.cuda.is_available():
    warn_if_untested()


# ----------------------------------------------------------------------------------------------------------------------
# layouts


def token_layout(x: torch.Tensor) -> TokenLayout:
    return TokenLayout(x.stride(0), x.stride(1), x.stride(2), x.shape[1], int(x.dtype == torch.float16))


def readable(x: torch.Tensor) -> torch.Tensor:
    """x itself if the kernels can read it in place (contiguous last dimension, 16-byte aligned tokens), else a
    contiguous copy (unica/__init__.py:103-108)."""
    in_place = (x.stride(-1) == 1 and x.data_ptr() % 16 == 0
                and all(x.stride(i) % 8 == 0 or x.shape[i] == 1 for i in range(3)))
    return x if in_place else x.contiguous()


def on_their_device(function):
    """Runs function(q, ...) with q's device current: launches go to that device's context and current stream."""

    @functools.wraps(function)
    def run(q, *args, **kwargs):
        with torch.cuda.device(q.device):
            return function(q, *args, **kwargs)

    return run


def _check_input(x: torch.Tensor, what: str) -> None:
    if not x.is_cuda:
        raise ValueError(f"{what} must be on the GPU")
    if x.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"{what} must be bfloat16 or float16, got {x.dtype}")
    if x.dim() != 4 or x.shape[-1] != HEAD_DIM:
        raise ValueError(f"{what} must be [batch, heads, tokens, {HEAD_DIM}], got {tuple(x.shape)}")
    if x.shape[2] == 0:
        raise ValueError(f"{what} must hold at least one token")


_status_words: dict = {}


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 word the attention kernels leave non-zero when one of their bounded waits gave up; one per device."""
    device = torch.device(device)
    if device not in _status_words:
        _status_words[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[device]


def check_status(device=None) -> None:
    """Synchronises and raises RuntimeError if a kernel reported a pipeline time-out since the last check.  The hot
    path never calls this (it would wait for the GPU); tests and the self-test do."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = status_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        raise RuntimeError(f"a unica-b200 kernel gave up waiting (status {code}, see common.cuh Status)")


# ----------------------------------------------------------------------------------------------------------------------
# statistics


def _stats(x: torch.Tensor, per: int, rope: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    batch, heads, n, _ = x.shape
    blocks = math.ceil(n / STATS_TOKENS)
    groups = 1 if per == 0 else math.ceil(n / per)
    partial = torch.empty(batch * heads, blocks, 3, HEAD_DIM, device=x.device)
    mean, low, high = (torch.empty(batch, heads, groups, HEAD_DIM, device=x.device) for _ in range(3))
    lib.call("unica_b200_channel_stats" + ("_rope" if rope is not None else ""), lib.ptr(x), token_layout(x), *rope_args(rope, x),
             batch * heads, n, per, lib.ptr(partial), lib.ptr(mean), lib.ptr(low), lib.ptr(high), lib.stream())
    return mean, low, high


@on_their_device
def block_stats(x: torch.Tensor, rope: torch.Tensor | None = None) -> torch.Tensor:
    """Sum, min and max per channel over each block of STATS_TOKENS tokens of x (rotated by rope first, if given):
    float32 [batch, heads, blocks, 3, 128] (unica/__init__.py:580-589).  rope_stats is this plus the reduction over blocks."""
    _check_input(x, "x")
    x = readable(x)
    batch, heads, n, _ = x.shape
    blocks = math.ceil(n / STATS_TOKENS)
    partial = torch.empty(batch * heads, blocks, 3, HEAD_DIM, device=x.device)
    scratch = torch.empty(3, batch, heads, 1, HEAD_DIM, device=x.device)
    lib.call("unica_b200_channel_stats" + ("_rope" if rope is not None else ""), lib.ptr(x), token_layout(x), *rope_args(rope, x),
             batch * heads, n, 0, lib.ptr(partial), lib.ptr(scratch[0]), lib.ptr(scratch[1]), lib.ptr(scratch[2]), lib.stream())
    return partial.view(batch, heads, blocks, 3, HEAD_DIM)


def wave_layout(heads: int, n_queries: int, n_keys: int, v_token: int, device) -> dict:
    """The reference picks between a 4-warp and an 8-warp block per call to fill its last wave (unica/__init__.py:281-285).
    Here every kernel has one block shape (accurate: one tile of 128 queries per block of 16 warps, one block per SM;
    fast: two query tiles per block of 12 warps), so there is nothing to pick: always {}.  What the last wave costs is
    what wave_plan() reports."""
    return {}


def wave_plan(heads: int, n_queries: int, kernel: str = DEFAULT_KERNEL, device=None) -> dict:
    """How a call's blocks fall on the SMs: blocks (all of equal length: every query tile meets every key), blocks per wave
    (one per SM), waves, and the share of the SM time of those waves that does work.  batch * heads for `heads`."""
    rows = 256 if kernel == "attention_fp4" else 128
    blocks = heads * math.ceil(n_queries / rows)
    per_wave = sm_count(torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device))
    waves = math.ceil(blocks / per_wave)
    return {"blocks": blocks, "per_wave": per_wave, "waves": waves, "efficiency": blocks / (waves * per_wave)}


def source(kernel: str, tile: dict) -> str:
    """The translation unit a call runs (the reference names the .cu file it builds, unica/__init__.py:256-261): the
    library is built ahead of time, every setting is a run-time argument."""
    _settings(kernel, tile)
    return "attention_fp4" if kernel == "attention_fp4" else "attention_int8"


@on_their_device
def rope_stats(x: torch.Tensor, rope: torch.Tensor | None = None, per: int | None = None):
    """Per channel of each head over all tokens of x: mean, min, max, float32 [batch, heads, 128]; with per (a multiple
    of 256) over each block of that many tokens, [batch, heads, blocks, 128] (unica/__init__.py:592-612).  One pass
    over x; sums in a fixed order, so the mean does not depend on how many heads the call holds.
    rope: ComfyUI's table (see rope_table); the statistics are then those of x rotated, which is never written."""
    _check_input(x, "x")
    if per is not None and per % STATS_TOKENS:
        raise ValueError(f"per must be a multiple of {STATS_TOKENS}, got {per}")
    mean, low, high = _stats(readable(x), per or 0, rope)
    return (mean, low, high) if per else (mean[:, :, 0], low[:, :, 0], high[:, :, 0])


# ----------------------------------------------------------------------------------------------------------------------
# RoPE inside the quantizers (unica/__init__.py:536-577)


def rope_table(rope: torch.Tensor, batch: int, n_queries: int, n_keys: int) -> torch.Tensor:
    """ComfyUI's RoPE table checked: float32 [batch or 1, tokens, 1, 64, 2, 2], self-attention."""
    if n_queries != n_keys:
        raise ValueError(f"rope= is for self-attention, got {n_queries} queries and {n_keys} keys")
    if (rope.dtype != torch.float32 or rope.dim() != 6 or rope.shape[1] != n_queries or rope.shape[2] != 1
            or rope.shape[3:] != (ROPE_PAIRS, 2, 2) or rope.shape[0] not in (1, batch)):
        raise ValueError(f"rope must be float32 [{batch} or 1, {n_queries}, 1, {ROPE_PAIRS}, 2, 2], "
                         f"got {rope.dtype} {tuple(rope.shape)}")
    return rope


# The table compacted last: (weak reference to it, its version, the compact table).  The blocks of a sampling step share
# one table, so it is converted once; a weak reference rather than an address, because the next step's table may be
# given the old one's memory.
_compact_rope: tuple = (lambda: None, -1, None)


def compact_rope(rope: torch.Tensor) -> torch.Tensor:
    """The table as the kernels read it: (cos, sin) per pair in fp16, [batch or 1, tokens, 64, 2].  The table must hold
    rotations [[c, -s], [s, c]].  Kept while the same table object, unmodified, comes back."""
    global _compact_rope
    version = None if rope.is_inference() else rope._version  # inference tensors have no version counter
    kept, kept_version, compact = _compact_rope
    if kept() is rope and kept_version == version:
        return compact
    cos, sin = rope[..., 0, 0], rope[..., 1, 0]
    if not (torch.equal(rope[..., 1, 1], cos) and torch.equal(rope[..., 0, 1], -sin)):
        raise ValueError("rope must hold rotations [[cos, -sin], [sin, cos]], as WAN's table does")
    compact = torch.stack([cos, sin], -1)[:, :, 0].half().contiguous()
    _compact_rope = (weakref.ref(rope), version, compact)
    return compact


def rope_args(rope: torch.Tensor | None, x: torch.Tensor) -> tuple:
    """The (table, batch stride) arguments of the *_rope entry points for x [batch, heads, tokens, 128]; () without rope."""
    if rope is None:
        return ()
    compact = compact_rope(rope_table(rope, x.shape[0], x.shape[2], x.shape[2]))
    if compact.device != x.device:
        raise ValueError(f"rope is on {compact.device}, the tensors on {x.device}")
    return lib.ptr(compact), compact.stride(0) if compact.shape[0] > 1 else 0


# ----------------------------------------------------------------------------------------------------------------------
# INT8 quantizers


@on_their_device
def quantize_int8(x: torch.Tensor, mean: torch.Tensor | None, block: int, rope: torch.Tensor | None = None,
                  tiles: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """x - mean ~ x8 * scale with one scale per `block` tokens over all of d (128: Q, 64: K); bit for bit the
    reference's quant() (unica/__init__.py:363-378).  mean: float32 [batch, heads, 128] or None.  rope: x is rotated
    first (mean is then the rotated x's).
    Returns int8 [batch, heads, tiles, 8, block, 16] (tile, 16-channel chunk, token, channel: the tcgen05 operand
    image; `decode_int8` gives [batch, heads, N, 128]) and float32 scales [batch, heads, tiles]."""
    _check_input(x, "x")
    x = readable(x)
    batch, heads, n, _ = x.shape
    need = math.ceil(n / block)
    tiles = need if tiles is None else tiles
    x8 = torch.empty(batch, heads, tiles, HEAD_DIM // 16, block, 16, dtype=torch.int8, device=x.device)
    scale = torch.empty(batch, heads, tiles, device=x.device)
    mean = None if mean is None else mean.float().contiguous()
    if block == Q_SCALE_BLOCK and mean is None and rope is None:  # the streaming form of the same kernel
        lib.call("unica_b200_quantize_q_int8_stream", lib.ptr(x), token_layout(x), batch * heads, n, tiles, lib.ptr(x8), lib.ptr(scale), lib.stream())
        return x8, scale
    lib.call("unica_b200_quantize_int8" + ("_rope" if rope is not None else ""), lib.ptr(x), token_layout(x), lib.ptr(mean),
             *rope_args(rope, x), batch * heads, n, block, tiles, lib.ptr(x8), lib.ptr(scale), lib.stream())
    return x8, scale


FUSED_SCRATCH_BYTES = 2 << 20  # include/unica_b200.h UNICA_B200_FUSED_SCRATCH_BYTES


@on_their_device
def quantize_k(k: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """K's mean over the tokens taken away and the rest in INT8 with a scale per 64 keys, in one launch that reads K from
    HBM once (unica_b200_quantize_k_int8_fused): what rope_stats(k)[0] and quantize_int8(k, mean, 64) give, except that
    the mean's terms are added in another (fixed) order.  Returns codes, scales, mean [batch, heads, 128]."""
    _check_input(k, "k")
    k = readable(k)
    batch, heads, n, _ = k.shape
    tiles = math.ceil(n / K_SCALE_BLOCK)
    k8 = torch.empty(batch, heads, tiles, HEAD_DIM // 16, K_SCALE_BLOCK, 16, dtype=torch.int8, device=k.device)
    scale = torch.empty(batch, heads, tiles, device=k.device)
    mean = torch.empty(batch, heads, HEAD_DIM, device=k.device)
    scratch = torch.empty(FUSED_SCRATCH_BYTES, dtype=torch.uint8, device=k.device)
    lib.call("unica_b200_quantize_k_int8_fused", lib.ptr(k), token_layout(k), batch * heads, n, tiles, lib.ptr(scratch), FUSED_SCRATCH_BYTES,
             lib.ptr(k8), lib.ptr(scale), lib.ptr(mean), lib.ptr(status_word(k.device)), lib.stream())
    return k8, scale, mean


@on_their_device
def quantize_v_channel(v: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """quantize_v(v) with its statistics pass folded in (unica_b200_quantize_v_int8_fused): the same bits, V read from HBM
    once."""
    _check_input(v, "v")
    v = readable(v)
    batch, heads, n, _ = v.shape
    tiles = math.ceil(n / V8_PAD_KEYS)
    v8 = torch.empty(batch, heads, tiles, 4, HEAD_DIM, 16, dtype=torch.int8, device=v.device)
    scale = torch.empty(batch, heads, HEAD_DIM, device=v.device)
    scratch = torch.empty(FUSED_SCRATCH_BYTES, dtype=torch.uint8, device=v.device)
    lib.call("unica_b200_quantize_v_int8_fused", lib.ptr(v), token_layout(v), batch * heads, n, lib.ptr(scratch), FUSED_SCRATCH_BYTES,
             lib.ptr(v8), lib.ptr(scale), lib.ptr(status_word(v.device)), lib.stream())
    return v8, scale


def decode_int8(x8: torch.Tensor, n: int) -> torch.Tensor:
    """quantize_int8's codes as plain int8 [batch, heads, n, 128]."""
    batch, heads, tiles, chunks, block, _ = x8.shape
    return x8.permute(0, 1, 2, 4, 3, 5).reshape(batch, heads, tiles * block, HEAD_DIM)[:, :, :n]


@on_their_device
def quantize_v(v: torch.Tensor, layout: int = 2, per_token: bool = False, outliers: int = 0) -> tuple[torch.Tensor, ...]:
    """v ~ v8 * scale (unica/__init__.py:402-444).  Per channel (default): one scale per channel over the head's
    tokens, float32 [batch, heads, 128].  per_token: one scale per token over its channels; returns v8, a scale of ones
    and float32 [batch, heads, tiles, 2, 64] = log2 s then 1 / s of each tile's keys (zeros past N).
    v8: int8 [batch, heads, tiles, 4, 128, 16] (tile, 16-key chunk, channel, key: the K-major operand of P.V);
    `decode_v8` gives [batch, heads, N, 128].  `layout` is accepted for compatibility: there is one layout here.
    outliers: the per-channel scale without the `outliers` (<= 8) keys of each head with the largest max |v|, which are
    written as zeros; returns v8, scale, those keys (int32 [batch, heads, outliers], -1: none) and their rows over the
    scale (float32 [batch, heads, outliers, 128]) for the kernel to add exactly."""
    if outliers and per_token:
        raise ValueError("per_token and outliers are two different V scales: pick one")
    if not 0 <= outliers <= MAX_OUTLIERS:
        raise ValueError(f"outliers must be in 0..{MAX_OUTLIERS}, got {outliers}")
    _check_input(v, "v")
    v = readable(v)
    batch, heads, n, _ = v.shape
    tiles = math.ceil(n / V8_PAD_KEYS)
    v8 = torch.empty(batch, heads, tiles, 4, HEAD_DIM, 16, dtype=torch.int8, device=v.device)
    scale = torch.empty(batch, heads, HEAD_DIM, device=v.device)
    low = high = tokens = skip = None
    if per_token:
        tokens = torch.empty(batch, heads, tiles, 2, V8_PAD_KEYS, device=v.device)
    elif outliers:
        keys = v_outliers(v, outliers)
        skip = torch.zeros(batch, heads, n, dtype=torch.uint8, device=v.device).scatter_(-1, keys, 1)
        partial = torch.empty(batch * heads, math.ceil(n / STATS_TOKENS), 3, HEAD_DIM, device=v.device)
        _, low, high = (torch.empty(batch, heads, HEAD_DIM, device=v.device) for _ in range(3))
        lib.call("unica_b200_channel_stats_masked", lib.ptr(v), token_layout(v), lib.ptr(skip), batch * heads, n,
                 lib.ptr(partial), lib.ptr(_), lib.ptr(low), lib.ptr(high), lib.stream())
    else:
        _, low, high = _stats(v, 0)
    lib.call("unica_b200_quantize_v_int8", lib.ptr(v), token_layout(v), lib.ptr(low), lib.ptr(high), lib.ptr(skip),
             int(per_token), batch * heads, n, lib.ptr(v8), lib.ptr(scale), lib.ptr(tokens), lib.stream())
    if per_token:
        return v8, scale, tokens
    if outliers:
        rows = v.gather(-2, keys[..., None].expand(-1, -1, -1, HEAD_DIM)).to(torch.bfloat16).float() / scale[..., None, :]
        missing = outliers - keys.shape[-1]  # fewer keys than outliers: the rest are none (-1) and zeros
        keys = torch.nn.functional.pad(keys, (0, missing), value=-1)
        rows = torch.nn.functional.pad(rows, (0, 0, 0, missing))
        return v8, scale, keys.int().contiguous(), rows.contiguous()
    return v8, scale


def v_outliers(v: torch.Tensor, count: int) -> torch.Tensor:
    """The `count` keys of each head with the largest max |v|, int64 [batch, heads, min(count, N)]
    (unica/__init__.py:384-390; the scale of the other keys comes from unica_b200_channel_stats_masked)."""
    low, high = torch.aminmax(v, dim=-1)  # per token, no copy of v
    return torch.maximum(high, -low).to(torch.bfloat16).float().topk(min(count, v.shape[-2]), -1).indices  # float16 counts as its bfloat16 rounding


def decode_v8(v8: torch.Tensor, n: int) -> torch.Tensor:
    """quantize_v's codes as plain int8 [batch, heads, n, 128]."""
    batch, heads, tiles = v8.shape[:3]
    return v8.permute(0, 1, 2, 3, 5, 4).reshape(batch, heads, tiles * V8_PAD_KEYS, HEAD_DIM)[:, :, :n]


# ----------------------------------------------------------------------------------------------------------------------
# the call


@on_their_device
def kernel_inputs(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel: str = DEFAULT_KERNEL,
                  rope: torch.Tensor | None = None, **tile: int) -> tuple:
    """The quantized operands `kernel` takes, apart from attention() so that quantization and kernel can be timed
    separately (unica/__init__.py:288-356)."""
    settings = _settings(kernel, tile)
    q, k, v = readable(q), readable(k), readable(v)
    if rope is not None:
        rope_table(rope, q.shape[0], q.shape[2], k.shape[2])
    q_tiles = 2 * math.ceil(q.shape[2] / (2 * Q_SCALE_BLOCK))  # the kernels take query tiles in pairs
    if kernel == "attention_fp4":  # Q and K in NVFP4 along d, V along the keys; Q smoothed per block of SMOOTH_Q queries
        smooth = settings["SMOOTH_Q"]
        if smooth % 256:
            raise ValueError(f"SMOOTH_Q must be a multiple of 256, got {smooth}")
        k_mean, k_low, k_high = rope_stats(k, rope)
        if smooth:
            q_mean, q_low, q_high = rope_stats(q, rope, smooth)
            q4, q_outer = quantize_fp4_rows(q, q_mean, 1, rope, (q_low, q_high), smooth, tiles=q_tiles)
            bias = smooth_bias(k, k_mean, q_mean, rope=rope)
        else:
            q4, q_outer = quantize_fp4_rows(q, None, 1, rope, tiles=q_tiles)
            bias = None
        k4, k_outer = quantize_fp4_rows(k, k_mean, 64, rope, (k_low, k_high))
        qk_outer = (q_outer * k_outer).clamp_min(1e-30).contiguous()
        v4, v_outer = quantize_v4(v)
        return q4, k4, v4, qk_outer, v_outer, bias, smooth
    q8, q_scale = quantize_int8(q, None, Q_SCALE_BLOCK, rope, tiles=q_tiles)
    if rope is None:  # statistics and quantizer in one launch
        k8, k_scale, _ = quantize_k(k)
    else:
        k_mean = rope_stats(k, rope)[0]  # softmax cancels the mean
        k8, k_scale = quantize_int8(k, k_mean, K_SCALE_BLOCK, rope)
    if settings["V_TOKEN"]:
        v8, v_scale, v_token = quantize_v(v, per_token=True)
        return q8, q_scale, k8, k_scale, v8, v_scale, v_token, lib.V_TOKEN
    if settings["V_OUTLIERS"]:
        v8, v_scale, keys, rows = quantize_v(v, outliers=settings["V_OUTLIERS"])
        return q8, q_scale, k8, k_scale, v8, v_scale, (keys, rows), lib.V_OUTLIERS
    v8, v_scale = quantize_v_channel(v)
    return q8, q_scale, k8, k_scale, v8, v_scale, None, lib.V_CHANNEL


def _settings(kernel: str, tile: dict) -> dict:
    if kernel not in KERNELS:
        raise ValueError(f"unknown kernel {kernel!r}, expected one of {KERNELS}")
    if unknown := tile.keys() - TILE.keys():
        raise ValueError(f"unknown tile settings {sorted(unknown)}, expected some of {sorted(TILE)}")
    settings = TILE | tile
    if settings["KEYS_PER_TILE"] != KEYS_PER_TILE:
        raise ValueError(f"KEYS_PER_TILE is fixed at {KEYS_PER_TILE}: it is part of the numerics")
    return settings


@on_their_device
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel: str = DEFAULT_KERNEL,
              inputs: tuple | None = None, rope: torch.Tensor | None = None, out: torch.Tensor | None = None,
              peer_out: Sequence[int] = (), **tile: int) -> torch.Tensor:
    """softmax(q k^T / sqrt(d)) v, non-causal.  q [batch, heads, n_queries, 128]; k, v [batch, heads, n_keys, 128]; all
    bfloat16 or all float16, on a B200.  Returns a tensor like q (dtype and strides).  kernel / tile pick the mode, as
    in PRESETS.  inputs: what kernel_inputs() returned for these q, k, v; the kernel then runs alone.
    float16 tensors are read as they are, each element rounded to bfloat16 on its way into the quantizers: the result is
    bit for bit that of converting q, k, v first (what the reference does), without the copies.
    out: where to write, a tensor of q's shape and dtype (any strides the kernels can address: see readable()), returned.
    peer_out: with out, up to 7 device addresses of tensors laid out like out in other GPUs' memory, mapped into this
    process; the kernel stores every row there as well (see shard.SharedOutput, which also does the barriers this needs).
    Same checks and exceptions as the reference (unica/__init__.py:126-190)."""
    settings = _settings(kernel, tile)
    if out is not None:
        if out.dtype != q.dtype or out.shape != q.shape or out.device != q.device or readable(out) is not out:
            raise ValueError("out must be a tensor of q's shape and dtype on q's device, 16-byte aligned rows with contiguous channels")
    elif peer_out:
        raise ValueError("peer_out needs out")
    if not (q.dtype == k.dtype == v.dtype and q.dtype in (torch.bfloat16, torch.float16)):
        raise TypeError(f"q, k, v must all be bfloat16 or all float16, got {q.dtype}, {k.dtype}, {v.dtype}")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("q, k, v must be on the GPU")
    if q.dim() != 4 or q.shape[-1] != HEAD_DIM:
        raise ValueError(f"q must be [batch, heads, tokens, {HEAD_DIM}], got {tuple(q.shape)}")
    if k.shape != v.shape or k.shape[:2] != q.shape[:2] or k.shape[-1] != HEAD_DIM:
        raise ValueError(f"k and v must be [batch, heads, n_keys, {HEAD_DIM}] like q, "
                         f"got q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    batch, heads, n_queries, _ = q.shape
    n_keys = k.shape[2]
    if n_keys == 0:
        raise ValueError("k and v must hold at least one token")
    if rope is not None:
        rope_table(rope, batch, n_queries, n_keys)
    if inputs is None and heads_per_call(q, k, kernel, tile) < heads:
        return in_pieces(q, k, v, kernel, rope, tile, out, peer_out)
    q, k, v = readable(q), readable(k), readable(v)
    if out is None:
        out = torch.empty_like(q)
    peers = (ctypes.c_void_p * len(peer_out))(*peer_out) if peer_out else None
    if n_queries == 0:
        return out
    if inputs is None:
        try:
            inputs = kernel_inputs(q, k, v, kernel, rope, **tile)
        except torch.cuda.OutOfMemoryError:
            # The planner's picture of free memory was out of date (something took memory since it asked): forget it and
            # go by heads, fewer than before, on what is free now.
            _FREE_VRAM.pop(q.device, None)
            torch.cuda.empty_cache()
            if heads == 1:
                raise
            return in_pieces(q, k, v, kernel, rope, tile, out, peer_out, max(1, min(heads // 2, heads_per_call(q, k, kernel, tile))))
    if kernel == "attention_fp4":
        q4, k4, v4, qk_outer, v_outer, bias, smooth = inputs
        lib.call("unica_b200_attention_fp4_peers", lib.ptr(q4.codes), lib.ptr(q4.sf), lib.ptr(k4.codes), lib.ptr(k4.sf),
                 lib.ptr(v4.codes), lib.ptr(v4.sf), lib.ptr(qk_outer), lib.ptr(v_outer), lib.ptr(bias),
                 0 if bias is None else bias.shape[2], smooth, lib.ptr(out), peers, len(peer_out), token_layout(out), batch * heads,
                 n_queries, n_keys, HEAD_DIM**-0.5 * LOG2E, lib.ptr(status_word(q.device)), lib.stream())
        return out
    q8, q_scale, k8, k_scale, v8, v_scale, v_token, v_mode = inputs
    keys, rows = v_token if v_mode == lib.V_OUTLIERS else (None, None)
    lib.call("unica_b200_attention_int8_peers", lib.ptr(q8), lib.ptr(q_scale), lib.ptr(k8), lib.ptr(k_scale), lib.ptr(v8),
             lib.ptr(v_scale), lib.ptr(v_token if v_mode == lib.V_TOKEN else None), v_mode, lib.ptr(keys), lib.ptr(rows),
             0 if keys is None else keys.shape[-1], lib.ptr(out), peers, len(peer_out), token_layout(out), batch * heads, n_queries,
             n_keys, HEAD_DIM**-0.5 * LOG2E, lib.ptr(status_word(q.device)), lib.stream())
    del settings
    return out


# ----------------------------------------------------------------------------------------------------------------------
# the head-split planner (unica/__init__.py:193-245): on a 180 GB part it rarely splits, but the contract stays


_FREE_VRAM: dict = {}  # device -> (bytes free, when asked)
FREE_VRAM_MAX_AGE = 0.25  # seconds: the driver's answer costs 0.1 to 1 ms of host time, too much to pay on every call
STALE_FRACTION = 8  # ... but a call that needs more than an eighth of what was free then asks again (weights may have come in since)


def free_vram(device: torch.device, fresh: bool = False) -> int:
    """Bytes the driver has free on the device (plus what torch's allocator holds unused); does not wait for the GPU.
    The driver is asked at most every FREE_VRAM_MAX_AGE seconds per device, unless `fresh`."""
    now = time.monotonic()
    cached = _FREE_VRAM.get(device)
    if fresh or cached is None or now - cached[1] > FREE_VRAM_MAX_AGE:
        free, _ = torch.cuda.mem_get_info(device)
        cached = _FREE_VRAM[device] = (free, now)
    return cached[0]


def vram_reserve(device: torch.device) -> int:
    if VRAM_RESERVE is not None:
        return VRAM_RESERVE
    return max(2**30, torch.cuda.get_device_properties(device).total_memory // 10)


def heads_per_call(q: torch.Tensor, k: torch.Tensor, kernel: str, tile: dict) -> int:
    """How many heads one call takes without its temporary buffers reaching the reserve.  Per head: the quantized q, k,
    v and the output, at most 2 bytes per element of q, k, v (float16 inputs are read in place, like bfloat16); in the fast
    mode the smoothing table, one float per key and block of SMOOTH_Q queries (unica/__init__.py:208-232 counts the same
    things).  A small call runs whole."""
    batch, heads, n_queries, _ = q.shape
    n_keys = k.shape[2]
    elements = batch * HEAD_DIM * (n_queries + 2 * n_keys)
    per_head = max(1, elements * 2)
    smooth = (TILE | tile).get("SMOOTH_Q", 0) if kernel == "attention_fp4" else 0
    if smooth:
        per_head += batch * 4 * math.ceil(n_queries / smooth) * n_keys
    free, reserve = free_vram(q.device), vram_reserve(q.device)
    if heads * per_head > free // STALE_FRACTION:  # a call this size must not trust an answer something else may have outdated
        free = free_vram(q.device, fresh=True)
    if heads * per_head <= min(reserve // SMALL_CALL_FRACTION, free):
        step = heads
    else:
        step = max(1, min(heads, (free - reserve) // per_head))
    if LOG_VRAM:
        print(f"[unica vram] tokens {n_queries} heads {heads} {q.dtype} driver_free {free / 2**30:.2f} "
              f"reserve {reserve / 2**30:.2f} per_head {per_head / 2**30:.3f} GiB -> {step} heads per call", flush=True)
    return step


def in_pieces(q, k, v, kernel: str, rope, tile: dict, out: torch.Tensor | None = None, peer_out: Sequence[int] = (),
              step: int | None = None) -> torch.Tensor:
    """attention() a few heads at a time into one output in q's dtype and layout (or into `out` and its peers, piece by
    piece).  Every head has its own statistics and scales, summed in a
    fixed order, so the result is bit for bit that of one call."""
    step = step or heads_per_call(q, k, kernel, tile)
    if out is not None:
        for first in range(0, q.shape[1], step):
            piece = slice(first, first + step)
            ahead = first * out.stride(1) * out.element_size()
            attention(q[:, piece], k[:, piece], v[:, piece], kernel, None, rope, out[:, piece], [p + ahead for p in peer_out], **tile)
        return out
    out = torch.empty_like(q)
    if readable(out) is not out:  # q in a layout the kernels cannot write: pieces through temporaries
        for first in range(0, q.shape[1], step):
            piece = slice(first, first + step)
            out[:, piece] = attention(q[:, piece], k[:, piece], v[:, piece], kernel, None, rope, **tile)
        return out
    return in_pieces(q, k, v, kernel, rope, tile, out, (), step)


_SM_COUNTS: dict = {}


def sm_count(device: torch.device) -> int:
    if device not in _SM_COUNTS:
        _SM_COUNTS[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNTS[device]


from unicaattention_b200.fp4 import (FP4V, FP4Rows, decode_fp4_rows, decode_v4, quantize_fp4_rows, quantize_v4,  # noqa: E402,F401
                                     smooth_bias)
from unicaattention_b200.host import attention_host  # noqa: E402,F401
