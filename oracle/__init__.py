"""CPU oracle for the quantized-attention forward path: ctypes wrapper over unica_oracle.c.

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by the smoke check and by the benchmark's CPU-baseline leg; the product
package never imports it.  The arithmetic restates the reference's emulator (bench/emulate.py) and quantizer kernels
(csrc/flash.cu); see the header of unica_oracle.c for the function-by-function citations.

Pinned: with recip=False every quantizer here equals the reference emulator run on CPU tensors bit for bit, and the
attention outputs agree to float rounding (tests/golden/, made by tests/golden/make_golden.py from the reference).

Arrays are numpy, contiguous [heads, tokens, 128]; bf16 inputs are uint16 bit patterns (see `bf16_bits`).
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libunica_oracle.so"
D = 128
TILE = 64
V_CHANNEL, V_TOKEN, V_OUTLIERS = 0, 1, 2
E2M1_VALUES = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def build(force: bool = False) -> Path:
    """Compile unica_oracle.c if the library is missing or older than the source."""
    src = HERE / "unica_oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "libunica_oracle.so"], check=True, capture_output=True)
    return LIB


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(LIB))
        _lib.uo_e4m3_to_float.restype = ctypes.c_float
        _lib.uo_e2m1_to_float.restype = ctypes.c_float
        _lib.uo_float_to_e4m3.argtypes = [ctypes.c_float]
        _lib.uo_float_to_e2m1.argtypes = [ctypes.c_float]
        _lib.uo_float_to_e4m3.restype = ctypes.c_uint8
        _lib.uo_float_to_e2m1.restype = ctypes.c_uint8
    return _lib


def threads(n: int = 0) -> int:
    """Host threads the OpenMP loops use; n > 0 sets them first (a launcher such as torchrun starts its workers with
    OMP_NUM_THREADS=1)."""
    return int(lib().uo_set_threads(int(n)))


def bf16_bits(x) -> np.ndarray:
    """A torch bfloat16 tensor (any device) or a float array as contiguous uint16 bf16 bit patterns [heads, n, 128]."""
    if hasattr(x, "detach"):  # torch tensor
        import torch

        x = x.detach().to("cpu")
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        x = x.contiguous().view(torch.int16).numpy().view(np.uint16)
    else:
        x = np.ascontiguousarray(x)
        if x.dtype != np.uint16:
            u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
            x = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.ascontiguousarray(x.reshape(-1, x.shape[-2], D))


def bf16_to_float(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a, shape=None):
    if a is None:
        return None
    if hasattr(a, "detach"):
        a = a.detach().float().cpu().numpy()
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a if shape is None else a.reshape(shape)


def wan_rope_table(t: int, h: int, w: int, dim: int = D, theta: float = 10000.0) -> np.ndarray:
    """The RoPE table of a t x h x w video latent as WAN models get it from ComfyUI (axes of 44, 42 and 42 channels for
    d = 128; the reference's tests use bench/emulate.py:133-143): float32 [1, t * h * w, 1, 64, 2, 2], a rotation
    [[cos, -sin], [sin, cos]] per pair of channels."""
    axes = [dim - 4 * (dim // 6), 2 * (dim // 6), 2 * (dim // 6)]
    ids = np.stack(np.meshgrid(np.arange(t), np.arange(h), np.arange(w), indexing="ij"), -1).reshape(-1, 3)
    tables = []
    for axis, size in enumerate(axes):
        omega = 1.0 / theta ** np.linspace(0, (size - 2) / size, size // 2, dtype=np.float64)
        angle = ids[:, axis, None].astype(np.float64) * omega  # [tokens, size / 2]
        tables.append(np.stack([np.cos(angle), -np.sin(angle), np.sin(angle), np.cos(angle)], -1).reshape(-1, size // 2, 2, 2))
    return np.concatenate(tables, 1).astype(np.float32)[None, :, None]


def _rope(rope, heads: int):
    """(cos, sin) float32 [tables, n, 64, 2] rounded to fp16, and how many heads share a table; (None, 1) without rope.
    rope: ComfyUI's table [batch or 1, n, 1, 64, 2, 2] (torch or numpy)."""
    if rope is None:
        return None, 1
    if hasattr(rope, "detach"):
        rope = rope.detach().float().cpu().numpy()
    rope = np.asarray(rope, dtype=np.float32)
    compact = np.stack([rope[:, :, 0, :, 0, 0], rope[:, :, 0, :, 1, 0]], -1)  # [tables, n, 64, 2]
    compact = np.ascontiguousarray(compact.astype(np.float16).astype(np.float32))
    assert heads % compact.shape[0] == 0
    return compact, heads // compact.shape[0]


def rope_rotate(x, rope) -> np.ndarray:
    """x rotated in float as the quantizers do it: float32 [heads, n, 128], not rounded to bf16."""
    x = bf16_bits(x)
    heads, n, _ = x.shape
    table, per = _rope(rope, heads)
    out = np.empty((heads, n, D), np.float32)
    lib().uo_rope(_p(x), _p(table), per, heads, n, _p(out))
    return out


def slot_key() -> np.ndarray:
    """slot -> key inside a 64-key tile (the fast mode's key order)."""
    return np.array([lib().uo_slot_key(s) for s in range(TILE)], dtype=np.int64)


def channel_stats(x, per: int = 0, rope=None):
    """mean, min, max per channel over each group of `per` tokens (0: the head): float32 [heads, groups, 128]."""
    x = bf16_bits(x)
    heads, n, _ = x.shape
    groups = 1 if per <= 0 else -(-n // per)
    mean, low, high = (np.empty((heads, groups, D), np.float32) for _ in range(3))
    table, shared = _rope(rope, heads)
    lib().uo_channel_stats_rope(_p(x), _p(table), shared, heads, n, per, _p(mean), _p(low), _p(high))
    return mean, low, high


def quantize_int8(x, mean, block: int, recip: bool = True, rope=None):
    x = bf16_bits(x)
    heads, n, _ = x.shape
    mean = _f32(mean, (heads, D))
    codes = np.empty((heads, n, D), np.int8)
    scales = np.empty((heads, -(-n // block)), np.float32)
    table, shared = _rope(rope, heads)
    lib().uo_quantize_int8_rope(_p(x), _p(mean), _p(table), shared, heads, n, block, int(recip), _p(codes), _p(scales))
    return codes, scales


def quantize_v_channel(v, skip=None, recip: bool = True):
    v = bf16_bits(v)
    heads, n, _ = v.shape
    if skip is not None:
        skip = np.ascontiguousarray(skip, dtype=np.uint8).reshape(heads, n)
    codes = np.empty((heads, n, D), np.int8)
    scale = np.empty((heads, D), np.float32)
    lib().uo_quantize_v_channel(_p(v), _p(skip), heads, n, int(recip), _p(codes), _p(scale))
    return codes, scale


def quantize_v_token(v, recip: bool = True):
    v = bf16_bits(v)
    heads, n, _ = v.shape
    codes = np.empty((heads, n, D), np.int8)
    s, log_s, inv_s = (np.empty((heads, n), np.float32) for _ in range(3))
    lib().uo_quantize_v_token(_p(v), heads, n, int(recip), _p(codes), _p(s), _p(log_s), _p(inv_s))
    return codes, s, log_s, inv_s


def v_outlier_keys(v, count: int):
    v = bf16_bits(v)
    heads, n, _ = v.shape
    keys = np.empty((heads, count), np.int32)
    lib().uo_v_outlier_keys(_p(v), heads, n, count, _p(keys))
    return keys


def nvfp4_rows(x, mean=None, mean_tokens: int = 0, recip: bool = True, rope=None):
    """codes uint8 [heads, n, 128] (4-bit codes), e4m3 scale bytes [heads, n, 8], outer float32 [heads]."""
    x = bf16_bits(x)
    heads, n, _ = x.shape
    groups = 1 if mean_tokens <= 0 else -(-n // mean_tokens)
    mean = _f32(mean, (heads, groups, D))
    codes = np.empty((heads, n, D), np.uint8)
    sf = np.empty((heads, n, 8), np.uint8)
    outer = np.empty((heads,), np.float32)
    table, shared = _rope(rope, heads)
    lib().uo_nvfp4_rows_rope(_p(x), _p(mean), mean_tokens, _p(table), shared, heads, n, int(recip), _p(codes), _p(sf), _p(outer))
    return codes, sf, outer


def nvfp4_v(v, recip: bool = True):
    """codes uint8 [heads, tiles * 64, 128] by slot position, scale bytes [heads, tiles, 4, 128], outer [heads, 128]."""
    v = bf16_bits(v)
    heads, n, _ = v.shape
    tiles = -(-n // TILE)
    codes = np.empty((heads, tiles * TILE, D), np.uint8)
    sf = np.empty((heads, tiles, 4, D), np.uint8)
    outer = np.empty((heads, D), np.float32)
    lib().uo_nvfp4_v(_p(v), heads, n, int(recip), _p(codes), _p(sf), _p(outer))
    return codes, sf, outer


def _rows(nq, q_first, q_count):
    if q_count is None:
        q_count = nq - q_first
    assert 0 <= q_first and q_first + q_count <= nq
    return q_first, q_count


def reference_fp32(q, k, v, q_first: int = 0, q_count: int | None = None, rope=None) -> np.ndarray:
    """softmax(q k^T / sqrt(d)) v in float (double accumulation): float32 [heads, q_count, 128], not rounded."""
    q, k, v = bf16_bits(q), bf16_bits(k), bf16_bits(v)
    heads, nq, _ = q.shape
    q_first, q_count = _rows(nq, q_first, q_count)
    out = np.empty((heads, q_count, D), np.float32)
    table, shared = _rope(rope, heads)
    lib().uo_reference_fp32_rope(_p(q), _p(k), _p(v), _p(table), shared, heads, nq, k.shape[1], q_first, q_count, _p(out))
    return out


def attention_accurate(q, k, v, v_mode: int = V_CHANNEL, outliers: int = 8, recip: bool = True, k_mean=None,
                       q_first: int = 0, q_count: int | None = None, rope=None) -> np.ndarray:
    """The accurate mode's contract; float32 [heads, q_count, 128] already rounded to bf16."""
    q, k, v = bf16_bits(q), bf16_bits(k), bf16_bits(v)
    heads, nq, _ = q.shape
    q_first, q_count = _rows(nq, q_first, q_count)
    k_mean = _f32(k_mean, (heads, D))
    out = np.empty((heads, q_count, D), np.float32)
    table, shared = _rope(rope, heads)
    lib().uo_attention_accurate_rope(_p(q), _p(k), _p(v), _p(table), shared, heads, nq, k.shape[1], v_mode, outliers, int(recip),
                                     _p(k_mean), q_first, q_count, _p(out))
    return out


def attention_fast(q, k, v, smooth_q: int = 512, recip: bool = True, k_mean=None, q_mean=None, q_first: int = 0,
                   q_count: int | None = None, rope=None) -> np.ndarray:
    """The fast mode's contract; float32 [heads, q_count, 128] already rounded to bf16."""
    q, k, v = bf16_bits(q), bf16_bits(k), bf16_bits(v)
    heads, nq, _ = q.shape
    q_first, q_count = _rows(nq, q_first, q_count)
    k_mean = _f32(k_mean, (heads, D))
    if q_mean is not None:
        q_mean = _f32(q_mean, (heads, -(-nq // smooth_q), D))
    out = np.empty((heads, q_count, D), np.float32)
    table, shared = _rope(rope, heads)
    lib().uo_attention_fast_rope(_p(q), _p(k), _p(v), _p(table), shared, heads, nq, k.shape[1], smooth_q, int(recip), _p(k_mean),
                                 _p(q_mean), q_first, q_count, _p(out))
    return out


def attention_fast_codes(q, k, v, smooth_q: int = 512, recip: bool = True, k_mean=None, q_mean=None):
    """attention_fast() over all rows, and the quantized probabilities it formed on the way: (out, codes uint8
    [heads, nq, tiles, 64] in slot order, scale bytes uint8 [heads, nq, tiles, 4])."""
    q, k, v = bf16_bits(q), bf16_bits(k), bf16_bits(v)
    heads, nq, _ = q.shape
    tiles = -(-k.shape[1] // 64)
    k_mean = _f32(k_mean, (heads, D))
    if q_mean is not None:
        q_mean = _f32(q_mean, (heads, -(-nq // smooth_q), D))
    out = np.empty((heads, nq, D), np.float32)
    record = np.zeros((heads, nq, tiles, 68), np.uint8)
    lib().uo_attention_fast_codes(_p(q), _p(k), _p(v), heads, nq, k.shape[1], smooth_q, int(recip), _p(k_mean), _p(q_mean), _p(out),
                                  _p(record))
    return out, record[..., :64], record[..., 64:]


def rel_l2(a, b) -> float:
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm((a - b).ravel()) / np.linalg.norm(b.ravel()))
