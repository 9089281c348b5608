"""The NVFP4 quantizers and the smoothing term against the oracle: codes, scale bytes and outer scales bit for bit
(the reference's tests/test_fp4.py:51-75, 102-115), through the C ABI."""

import numpy as np
import pytest
import torch

import oracle
from gpu_common import np_heads, randn_bf16

pytestmark = pytest.mark.gpu


def dequant(codes, sf_per_element_block, outer):
    """codes [..., 128 or n], scale bytes already broadcast per element -> float32 values code * (e4m3 * outer)."""
    scales = torch.from_numpy(np.ascontiguousarray(sf_per_element_block)).view(torch.float8_e4m3fn).float().numpy() * outer
    return oracle.E2M1_VALUES[codes] * scales


def rows_case(n, seed):
    x = randn_bf16((1, 3, n, 128), seed)
    x = x.float()
    x[..., :4] *= 30  # outlier channels
    x[0, 2] *= 1e-3  # a head far from 1
    return x.bfloat16()


@pytest.mark.parametrize("n", [1, 64, 1000, 1300])
def test_rows_bit_for_bit(n):
    import unicaattention_b200 as unica

    x = rows_case(n, n)
    xd = x.cuda()
    # K: minus the head mean, 64-key tiles in slot order
    k_mean = unica.rope_stats(xd)[0]
    k4, k_outer = unica.quantize_fp4_rows(xd, k_mean, 64)
    codes, sf = (np_heads(t) for t in unica.decode_fp4_rows(k4, n, slots=True))
    o_codes, o_sf, o_outer = oracle.nvfp4_rows(x, k_mean.cpu(), 0, recip=True)
    assert np.array_equal(np_heads(k_outer[..., None])[:, 0], o_outer)
    assert np.array_equal(sf, o_sf)
    live = np.repeat(o_sf, 16, -1) != 0  # a block whose scale is 0 holds zeros here, whatever the oracle's codes
    assert np.array_equal(codes[live], o_codes[live]) and not codes[~live].any()
    # Q: minus the mean of each block of 512 tokens, 128-query tiles, one more (empty) tile
    q_mean, low, high = unica.rope_stats(xd, None, 512)
    q4, q_outer = unica.quantize_fp4_rows(xd, q_mean, 1, None, (low, high), 512, tiles=-(-n // 128) + 1)
    codes, sf = (np_heads(t) for t in unica.decode_fp4_rows(q4, n))
    o_codes, o_sf, o_outer = oracle.nvfp4_rows(x, q_mean.cpu(), 512, recip=True)
    assert np.array_equal(np_heads(q_outer[..., None])[:, 0], o_outer)
    assert np.array_equal(sf, o_sf)
    live = np.repeat(o_sf, 16, -1) != 0
    assert np.array_equal(codes[live], o_codes[live])
    assert not q4.codes[:, :, -1].any() and not q4.sf[:, :, -1].any()
    # no mean at all
    p4, p_outer = unica.quantize_fp4_rows(xd, None)
    codes, sf = (np_heads(t) for t in unica.decode_fp4_rows(p4, n))
    o_codes, o_sf, o_outer = oracle.nvfp4_rows(x, None, 0, recip=True)
    assert np.array_equal(np_heads(p_outer[..., None])[:, 0], o_outer) and np.array_equal(sf, o_sf)


@pytest.mark.parametrize("n", [64, 1000, 4096, 7])
def test_v_bit_for_bit(n):
    import unicaattention_b200 as unica

    v = randn_bf16((1, 3, n, 128), 100 + n).float()
    v[0, 1] *= 1e-3
    v[..., :8] *= 40
    v = v.bfloat16()
    v4, outer = unica.quantize_v4(v.cuda())
    codes, sf = unica.decode_v4(v4)
    o_codes, o_sf, o_outer = oracle.nvfp4_v(v, recip=True)
    assert np.array_equal(np_heads(outer), o_outer)
    assert np.array_equal(np_heads(sf), o_sf)
    live = np.repeat(o_sf, 16, 2).reshape(o_codes.shape) != 0
    assert np.array_equal(np_heads(codes)[live], o_codes[live])
    # the rows of ones and their scales
    ones = v4.codes[:, :, :, :, 128:]
    second = v4.sf[:, :, :, 128:].unflatten(3, (32, 4))  # [.., lane, word, byte]: rows 128..143 are word 0 of lanes 0..15
    assert torch.all(ones == 0x22) and torch.all(second[:, :, :, :16, 0] == 0x38)
    assert not second[:, :, :, 16:].any() and not second[:, :, :, :, 1:].any()


def test_smooth_bias_is_exact_to_float():
    import unicaattention_b200 as unica

    g = torch.Generator().manual_seed(5)
    n = 1000
    q = torch.randn((2, 2, n, 128), generator=g) + 3 * torch.randn((2, 1, 128), generator=g) + \
        4 * torch.linspace(0, 1, n)[:, None] * torch.randn((2, 1, 128), generator=g)
    k = torch.randn((2, 2, n, 128), generator=g) + 0.3
    q, k = q.bfloat16().cuda(), k.bfloat16().cuda()
    q_mean = unica.rope_stats(q, None, 512)[0]
    k_mean = unica.rope_stats(k)[0]
    bias = unica.smooth_bias(k, k_mean, q_mean)
    assert bias.shape == (2, 2, 2, 1024)
    centred = k.double() - k_mean.double()[..., None, :]
    expected = (q_mean.double() @ centred.transpose(-1, -2)) * (128**-0.5 * 1.4426950408889634)  # [.., blocks, keys]
    slot_key = torch.tensor(unica.fp4.SLOT_KEY, device="cuda")
    order = (torch.arange(16, device="cuda")[:, None] * 64 + slot_key).flatten()  # position -> key
    valid = order < n
    got = bias[..., valid].double()
    want = expected[..., order[valid]]
    bound = (q_mean.abs().double() @ centred.abs().transpose(-1, -2))[..., order[valid]] * 2.0**-20 + 1e-6
    assert ((got - want).abs() <= bound).all(), ((got - want).abs() / bound).max()
    assert bool(torch.isneginf(bias[..., ~valid]).all())  # slots past the last key


def test_smooth_bias_many_query_blocks_and_an_odd_tile_count():
    """More than 64 query blocks (several passes of the kernel's 64 columns, the last one partly empty) and an odd number
    of key tiles (the last pair of tiles half empty)."""
    import unicaattention_b200 as unica

    g = torch.Generator().manual_seed(11)
    blocks, n_keys = 150, 3 * 64 - 7
    q_mean = torch.randn((1, 2, blocks, 128), generator=g).cuda() * torch.linspace(0.5, 2.0, blocks).cuda()[:, None]
    k = (torch.randn((1, 2, n_keys, 128), generator=g) + 0.5).bfloat16().cuda()
    k_mean = unica.rope_stats(k)[0]
    bias = unica.smooth_bias(k, k_mean, q_mean)
    unica.check_status()
    assert bias.shape == (1, 2, blocks, 192)
    centred = k.double() - k_mean.double()[..., None, :]
    expected = (q_mean.double() @ centred.transpose(-1, -2)) * (128**-0.5 * 1.4426950408889634)
    slot_key = torch.tensor(unica.fp4.SLOT_KEY, device="cuda")
    order = (torch.arange(3, device="cuda")[:, None] * 64 + slot_key).flatten()
    valid = order < n_keys
    got, want = bias[..., valid].double(), expected[..., order[valid]]
    bound = (q_mean.abs().double() @ centred.abs().transpose(-1, -2))[..., order[valid]] * 2.0**-20 + 1e-6
    assert ((got - want).abs() <= bound).all(), ((got - want).abs() / bound).max()
    assert bool(torch.isneginf(bias[..., ~valid]).all())
