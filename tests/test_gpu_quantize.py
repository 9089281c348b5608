"""The CUDA statistics and INT8 quantizers against the oracle: codes and scales bit for bit (the reference's
tests/test_quantize.py and tests/test_v_token.py:32-41), through the C ABI."""

import numpy as np
import pytest
import torch

import oracle
from gpu_common import np_heads, randn_bf16

pytestmark = pytest.mark.gpu
SHAPES = [(1, 2, 1000, 128), (2, 3, 77, 128), (1, 1, 128, 128), (1, 2, 1, 128), (1, 1, 700, 128)]


@pytest.mark.parametrize("shape", SHAPES)
def test_statistics(shape):
    import unicaattention_b200 as unica

    x = randn_bf16(shape, 5, channel_scale=True)
    mean, low, high = unica.rope_stats(x.cuda())
    o_mean, o_low, o_high = oracle.channel_stats(x)
    xf = np_heads(x)
    assert np.array_equal(np_heads(low), xf.min(1)) and np.array_equal(np_heads(high), xf.max(1))
    assert np.array_equal(np_heads(mean), o_mean[:, 0])  # same fixed order: bit for bit
    assert np.allclose(np_heads(mean), xf.mean(1, dtype=np.float64), atol=1e-6)
    if shape[2] > 256:
        mean, low, high = unica.rope_stats(x.cuda(), None, 512)
        o = oracle.channel_stats(x, 512)
        for got, want in zip((mean, low, high), o):
            assert np.array_equal(got.cpu().numpy().reshape(want.shape), want)
    with pytest.raises(ValueError):
        unica.rope_stats(x.cuda(), None, 100)
    # the per-block partials (the reference's block_stats): sums in the fixed lane order, minima and maxima exact
    partial = unica.block_stats(x.cuda()).cpu().numpy().reshape(-1, -(-shape[2] // 256), 3, 128)
    for b in range(partial.shape[1]):
        block = xf[:, 256 * b:256 * (b + 1)]
        assert np.array_equal(partial[:, b, 1], block.min(1)) and np.array_equal(partial[:, b, 2], block.max(1))
        assert np.allclose(partial[:, b, 0], block.sum(1, dtype=np.float64), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("shape", SHAPES)
def test_int8_rows_bit_for_bit(shape):
    import unicaattention_b200 as unica

    x = randn_bf16(shape, 0, channel_scale=True)
    xd = x.cuda()
    n = shape[2]
    mean = unica.rope_stats(xd)[0]
    for block, mu in ((128, None), (64, mean)):
        x8, scale = unica.quantize_int8(xd, mu, block)
        codes, scales = oracle.quantize_int8(x, None if mu is None else mu.cpu(), block, recip=True)
        assert np.array_equal(np_heads(scale), scales), (shape, block)
        assert np.array_equal(np_heads(unica.decode_int8(x8, n)), codes), (shape, block)
        # rows past the last token are zeros
        full = unica.decode_int8(x8, x8.shape[2] * block)
        assert not full[:, :, n:].any()
    # extra tiles (the attention kernel takes Q tiles in pairs) are zeros with the floor scale
    x8, scale = unica.quantize_int8(xd, None, 128, tiles=-(-n // 128) + 1)
    assert not x8[:, :, -1].any() and torch.all(scale[:, :, -1] == 1e-12)


@pytest.mark.parametrize("shape", SHAPES)
def test_v_bit_for_bit(shape):
    import unicaattention_b200 as unica

    v = randn_bf16(shape, 1, channel_scale=True)
    n = shape[2]
    v8, scale = unica.quantize_v(v.cuda())
    codes, scales = oracle.quantize_v_channel(v, recip=True)
    assert np.array_equal(np_heads(scale), scales)
    assert np.array_equal(np_heads(unica.decode_v8(v8, n)), codes)
    assert not unica.decode_v8(v8, v8.shape[2] * 64)[:, :, n:].any()
    v8, ones, tok = unica.quantize_v(v.cuda(), per_token=True)
    codes, s, log_s, inv_s = oracle.quantize_v_token(v, recip=True)
    assert torch.all(ones == 1)
    assert np.array_equal(np_heads(unica.decode_v8(v8, n)), codes)
    tok = tok.cpu().numpy().reshape(-1, tok.shape[2], 2, 64)
    got_log = tok[:, :, 0].reshape(tok.shape[0], -1)
    got_inv = tok[:, :, 1].reshape(tok.shape[0], -1)
    assert np.array_equal(got_inv[:, :n], inv_s)  # 1 / s is an IEEE division of a bit-exact s
    assert np.allclose(got_log[:, :n], log_s, rtol=0, atol=1e-6)
    assert not got_log[:, n:].any() and not got_inv[:, n:].any()


@pytest.mark.parametrize("shape", SHAPES)
def test_v_without_its_outlier_keys_bit_for_bit(shape):
    """The outliers scale: the 8 keys with the largest max |v| are zeros in V8 and take no part in the scale
    (the reference's tests/test_v_outliers.py compares its quantize_v(outliers=8) with its emulator the same way)."""
    import unicaattention_b200 as unica

    v = randn_bf16(shape, 5, channel_scale=True)
    n = shape[2]
    v[:, :, min(3, n - 1)] *= 40  # one key that would own the scale
    v8, scale, keys, rows = unica.quantize_v(v.cuda(), outliers=8)
    want_keys = oracle.v_outlier_keys(v, 8)
    got_keys = keys.cpu().numpy().reshape(-1, 8)
    assert np.array_equal(np.sort(got_keys, -1), np.sort(want_keys, -1))
    skip = np.zeros((want_keys.shape[0], n), dtype=np.uint8)
    for head, head_keys in enumerate(want_keys):
        skip[head, head_keys[head_keys >= 0]] = 1
    codes, scales = oracle.quantize_v_channel(v, skip, recip=True)
    assert np.array_equal(np_heads(scale), scales)
    assert np.array_equal(np_heads(unica.decode_v8(v8, n)), codes)
    vf = np_heads(v)
    for head in range(got_keys.shape[0]):
        for i, key in enumerate(got_keys[head]):
            want = vf[head, key] / scales[head] if key >= 0 else np.zeros(128, dtype=np.float32)
            assert np.array_equal(rows.cpu().numpy().reshape(-1, 8, 128)[head, i], want.astype(np.float32))
    with pytest.raises(ValueError):
        unica.quantize_v(v.cuda(), outliers=9)
    with pytest.raises(ValueError):
        unica.quantize_v(v.cuda(), per_token=True, outliers=8)


def test_strided_layout_is_read_in_place():
    """[batch, tokens, heads, 128] seen as [batch, heads, tokens, 128] (ComfyUI's layout) gives the same bytes
    (the reference's tests/test_attention.py:273-284, tests/test_v_token.py:62-68)."""
    import unicaattention_b200 as unica

    x = randn_bf16((2, 3, 300, 128), 7).cuda()
    strided = x.transpose(1, 2).contiguous().transpose(1, 2)
    assert strided.stride() != x.stride() and unica.readable(strided) is strided
    for a, b in zip(unica.quantize_int8(x, None, 128), unica.quantize_int8(strided, None, 128)):
        assert torch.equal(a, b)
    for a, b in zip(unica.quantize_v(x), unica.quantize_v(strided)):
        assert torch.equal(a, b)
