"""The fast mode's NVFP4 quantizers and smoothing term: host side of csrc/quantize_fp4.cu.

Same functions as the reference (`quantize_fp4_rows`, `quantize_v4`, `smooth_bias`, unica/__init__.py:452-521), with this
library's operand layouts (include/unica_b200.h); the `decode_*` helpers give back plain dequantized tensors for
comparisons with an emulation.
"""

from __future__ import annotations

import math
from typing import NamedTuple

import torch

from unicaattention_b200 import lib

HEAD_DIM = 128
FP4_TILE = 64
V4_ROWS, V4_SF_WORDS = 144, 256
LOG2E = 1.4426950408889634
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)
SLOT_KEY = tuple(32 * (k // 32) + 8 * (k % 8 // 2) + 2 * (k % 32 // 8) + k % 2 for k in range(64))  # slot -> key in a tile


class FP4Rows(NamedTuple):
    """Q or K in NVFP4: codes uint8 [batch, heads, tiles, 4, rows, 16]; scale bytes uint8, Q [batch, heads, tiles, 2, 128, 4],
    K [batch, heads, tiles, 32, 4, 4] (lane, word 2 step + row / 32, byte: the order tcgen05.cp takes)."""

    codes: torch.Tensor
    sf: torch.Tensor


class FP4V(NamedTuple):
    """V in NVFP4: codes uint8 [batch, heads, tiles, 2, 144, 16], scale bytes uint8 [batch, heads, tiles, 256, 4] (two blocks
    of 32 lanes x 4 words: channel c is word c / 32 of lane c % 32; the second block is the ones rows')."""

    codes: torch.Tensor
    sf: torch.Tensor


def _layout(x):
    return lib.TokenLayout(x.stride(0), x.stride(1), x.stride(2), x.shape[1], int(x.dtype == torch.float16))


def quantize_fp4_rows(x: torch.Tensor, mean: torch.Tensor | None, pad_to: int = 1, rope=None,
                      low_high: tuple[torch.Tensor, torch.Tensor] | None = None, mean_tokens: int | None = None,
                      tiles: int | None = None) -> tuple[FP4Rows, torch.Tensor]:
    """x - mean in NVFP4 along d under one float scale per head; bit for bit the reference emulator's
    block_scaled(x - mean, "nvfp4", -1).  pad_to 64: K (64-key tiles, keys in slot order); 1: Q (128-query tiles).
    mean: float32 [batch, heads, 128], or [batch, heads, blocks, 128] with mean_tokens (Q smoothing).  low_high: the
    per-channel (per block) min and max of x, as rope_stats returns them; taken here when not given.  rope: x is
    rotated first; mean and low_high are then the rotated x's.
    Returns (FP4Rows, outer float32 [batch, heads])."""
    import unicaattention_b200 as unica

    unica._check_input(x, "x")
    if pad_to not in (1, 64):
        raise ValueError(f"pad_to must be 1 (Q) or 64 (K), got {pad_to}")
    x = unica.readable(x)
    batch, heads, n, _ = x.shape
    rows = 64 if pad_to == 64 else 128
    per = mean_tokens or 0
    groups = 1 if not per else math.ceil(n / per)
    if low_high is None:
        _, low, high = unica._stats(x, per, rope)
    else:
        low, high = (t.float().reshape(batch, heads, groups, HEAD_DIM).contiguous() for t in low_high)
    mean_arg = None if mean is None else mean.float().reshape(batch, heads, groups, HEAD_DIM).contiguous()
    outer = torch.empty(batch, heads, device=x.device)
    lib.call("unica_b200_nvfp4_outer", lib.ptr(mean_arg), lib.ptr(low), lib.ptr(high), batch * heads, groups, lib.ptr(outer),
             lib.stream())
    need = math.ceil(n / rows)
    tiles = need if tiles is None else tiles
    codes = torch.empty(batch, heads, tiles, 4, rows, 16, dtype=torch.uint8, device=x.device)
    sf = torch.empty((batch, heads, tiles, 32, 4, 4) if rows == 64 else (batch, heads, tiles, 2, rows, 4), dtype=torch.uint8, device=x.device)
    lib.call("unica_b200_quantize_fp4_rows" + ("_rope" if rope is not None else ""), lib.ptr(x), _layout(x), lib.ptr(mean_arg), per,
             *unica.rope_args(rope, x), lib.ptr(outer), batch * heads, n, rows, tiles, lib.ptr(codes), lib.ptr(sf), lib.stream())
    return FP4Rows(codes, sf), outer


def quantize_v4(v: torch.Tensor) -> tuple[FP4V, torch.Tensor]:
    """V in NVFP4 along the keys, per channel, keys of each 64-key tile in slot order; bit for bit the reference
    emulator's block_scaled(slot_order(v), "nvfp4", -2, "channel").  Returns (FP4V, outer float32 [batch, heads, 128])."""
    import unicaattention_b200 as unica

    unica._check_input(v, "v")
    v = unica.readable(v)
    batch, heads, n, _ = v.shape
    tiles = math.ceil(n / FP4_TILE)
    _, low, high = unica._stats(v, 0)
    codes = torch.empty(batch, heads, tiles, 2, V4_ROWS, 16, dtype=torch.uint8, device=v.device)
    sf = torch.empty(batch, heads, tiles, V4_SF_WORDS, 4, dtype=torch.uint8, device=v.device)
    outer = torch.empty(batch, heads, HEAD_DIM, device=v.device)
    lib.call("unica_b200_quantize_v_fp4", lib.ptr(v), _layout(v), lib.ptr(low), lib.ptr(high), batch * heads, n, lib.ptr(codes),
             lib.ptr(sf), lib.ptr(outer), lib.stream())
    return FP4V(codes, sf), outer


def smooth_bias(k: torch.Tensor, k_mean: torch.Tensor, q_mean: torch.Tensor, qk_outer: torch.Tensor | None = None,
                padded_keys: int | None = None, rope=None) -> torch.Tensor:
    """The scores' share of Q's block means, added back exactly: q_mean[block] . (k - k_mean) to FP32 accuracy (on the
    tensor core, each value as two tf32 parts), times
    log2(e) / sqrt(128) (the attention kernel adds it to scores that are already in the log2 domain; the reference's
    table is divided by qk_outer instead, an argument kept here for the call's sake).  Keys of each 64-key tile in slot
    order, 0 past the last key.  Returns float32 [batch, heads, blocks, ceil64(n_keys)]."""
    import unicaattention_b200 as unica

    unica._check_input(k, "k")
    k = unica.readable(k)
    batch, heads, n, _ = k.shape
    blocks = q_mean.shape[2]
    padded = math.ceil(n / FP4_TILE) * FP4_TILE
    if padded_keys is not None and padded_keys != padded:
        raise ValueError(f"padded_keys must be {padded} for {n} keys, got {padded_keys}")
    bias = torch.empty(batch, heads, blocks, padded, device=k.device)
    lib.call("unica_b200_smooth_bias" + ("_rope" if rope is not None else ""), lib.ptr(k), _layout(k),
             lib.ptr(k_mean.float().contiguous()), lib.ptr(q_mean.float().contiguous()), *unica.rope_args(rope, k), batch * heads,
             blocks, n, HEAD_DIM**-0.5 * LOG2E, lib.ptr(bias), lib.ptr(unica.status_word(k.device)), lib.stream())
    return bias


# ----------------------------------------------------------------------------------------------------------------------
# decoding (tests, debugging)


def _nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., bytes] -> [..., 2 * bytes] 4-bit codes, low nibble first."""
    return torch.stack([codes & 0xF, codes >> 4], -1).flatten(-2)


def decode_fp4_rows(x4: FP4Rows, n: int, slots: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """(codes uint8 [batch, heads, n, 128], scale bytes uint8 [batch, heads, n, 8]) in token order."""
    codes, sf = x4
    batch, heads, tiles, _, rows, _ = codes.shape
    c = _nibbles(codes.permute(0, 1, 2, 4, 3, 5).reshape(batch, heads, tiles * rows, 64))  # [.., rows, 128]
    if rows == 64:  # K: [tiles, lane, (step, row / 32), byte] -> [tiles, row = 32 (row / 32) + lane, (step, byte)]
        s = sf.view(batch, heads, tiles, 32, 2, 2, 4).permute(0, 1, 2, 5, 3, 4, 6).reshape(batch, heads, tiles * rows, 8)
    else:
        s = sf.permute(0, 1, 2, 4, 3, 5).reshape(batch, heads, tiles * rows, 8)
    if slots:  # row r of a tile holds key slot_key(r): put the keys back in order
        key_of = torch.tensor(SLOT_KEY, device=codes.device)
        order = (torch.arange(tiles, device=codes.device)[:, None] * rows + key_of).flatten()
        inverse = torch.empty_like(order)
        inverse[order] = torch.arange(order.numel(), device=codes.device)
        c, s = c[:, :, inverse], s[:, :, inverse]
    return c[:, :, :n], s[:, :, :n]


def decode_v4(v4: FP4V) -> tuple[torch.Tensor, torch.Tensor]:
    """(codes uint8 [batch, heads, tiles * 64, 128] by slot position, scale bytes uint8 [batch, heads, tiles, 4, 128])."""
    codes, sf = v4
    batch, heads, tiles = codes.shape[:3]
    c = _nibbles(codes[:, :, :, :, :HEAD_DIM].permute(0, 1, 2, 4, 3, 5).reshape(batch, heads, tiles, HEAD_DIM, 32))  # [.., ch, 64 slots]
    c = c.transpose(-1, -2).reshape(batch, heads, tiles * FP4_TILE, HEAD_DIM)
    s = sf[:, :, :, :HEAD_DIM].view(batch, heads, tiles, 32, 4, 4).permute(0, 1, 2, 4, 3, 5).reshape(batch, heads, tiles, HEAD_DIM, 4)
    s = s.transpose(-1, -2)  # channel c = 32 (c / 32) + lane -> [.., tiles, 4, 128]
    return c, s


def probability_codes(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, smooth_q: int = 512) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The fast kernel run on bfloat16 q, k, v [batch, heads, tokens, 128] with its quantized probabilities kept
    (unica_b200_attention_fp4_codes): (out, e2m1 codes uint8 [batch, heads, n_queries, tiles, 64] in slot order, e4m3
    scale bytes uint8 [batch, heads, n_queries, tiles, 4]).  A diagnostic for tests, not a fast path."""
    import unicaattention_b200 as unica

    q, k, v = unica.readable(q), unica.readable(k), unica.readable(v)
    batch, heads, n_queries, _ = q.shape
    n_keys = k.shape[2]
    tiles = -(-n_keys // 64)
    q4, k4, v4, qk_outer, v_outer, bias, smooth = unica.kernel_inputs(q, k, v, "attention_fp4", SMOOTH_Q=smooth_q)
    out = torch.empty_like(q)
    words = torch.zeros((batch, heads, n_queries, tiles, 9), dtype=torch.int32, device=q.device)
    with torch.cuda.device(q.device):
        lib.call("unica_b200_attention_fp4_codes", lib.ptr(q4.codes), lib.ptr(q4.sf), lib.ptr(k4.codes), lib.ptr(k4.sf), lib.ptr(v4.codes),
                 lib.ptr(v4.sf), lib.ptr(qk_outer), lib.ptr(v_outer), lib.ptr(bias), 0 if bias is None else bias.shape[2], smooth,
                 lib.ptr(out), unica.token_layout(out), batch * heads, n_queries, n_keys, unica.HEAD_DIM**-0.5 * unica.LOG2E,
                 lib.ptr(words), lib.ptr(unica.status_word(q.device)), lib.stream())
    shifts = torch.arange(8, device=q.device, dtype=torch.int32) * 4
    codes = ((words[..., :8, None] >> shifts) & 15).to(torch.uint8).reshape(batch, heads, n_queries, tiles, 64)
    scale_bytes = ((words[..., 8:, None] >> (shifts[:4] * 2)) & 255).to(torch.uint8).reshape(batch, heads, n_queries, tiles, 4)
    return out, codes, scale_bytes
