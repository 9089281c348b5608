"""Pins the scale arithmetic the GPU kernels are held to.

torch divides a tensor by a Python number exactly on CPU tensors but as a multiplication by the reciprocal on CUDA
tensors; the reference kernels follow the CUDA form (csrc/flash.cu:355-357) and its bit-exact quantizer tests run the
emulator's pieces on CUDA tensors.  The golden vectors of tests/golden were made on the CPU, so they pin the oracle's
recip=False branch only.  Here the emulator's formulas (bench/emulate.py:36-47 token_scale, 52-60 to_fmt, 98-113
block_scaled) are written out with torch ON CUDA TENSORS, exactly as the emulator writes them, and both the kernels'
scales and the oracle's recip=True branch must equal them bit for bit.
"""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oracle
from gpu_common import np_heads, randn_bf16

pytestmark = pytest.mark.gpu
SHAPES = [(1, 4, 1024, 128), (2, 3, 77, 128), (1, 2, 1000, 128)]


def token_scale(x, block, qmax):
    """bench/emulate.py:36-47, verbatim arithmetic: one scale per block of tokens over all of d, [..., N]."""
    n = x.shape[-2]
    a = x.abs().amax(-1)
    a = F.pad(a, (0, -n % block)).unflatten(-1, (-1, block)).amax(-1, keepdim=True)
    a = a.expand(*a.shape[:-1], block).flatten(-2)[..., :n]
    return (a / qmax).clamp_min(1e-12)


def test_cuda_division_by_a_number_is_a_reciprocal_multiply():
    """The premise itself, checked once on this box's torch: a / 127.0 on a CUDA tensor is a * (1 / 127.0), not the
    IEEE quotient (which differs in the last bit for a few per cent of the values)."""
    g = torch.Generator().manual_seed(0)
    a = (torch.rand(1 << 20, generator=g) * 8).cuda()
    for number in (127.0, 6.0, 6.0 * 448.0):
        got = a / number
        assert torch.equal(got, a * torch.tensor(1.0 / number, dtype=torch.float32, device="cuda"))
        exact = (a.double() / number).float()
        assert 0 < (got != exact).float().mean().item() < 0.5


@pytest.mark.parametrize("shape", SHAPES)
def test_int8_scales_and_codes(shape):
    import unicaattention_b200 as unica

    x = randn_bf16(shape, 11, channel_scale=True)
    xd = x.cuda()
    n = shape[2]
    k_mean = unica.rope_stats(xd)[0]
    for block, mean in ((128, None), (64, k_mean)):
        centred = xd.float() if mean is None else xd.float() - mean[..., None, :]
        s = token_scale(centred, block, 127.0)  # [b, h, n]
        codes = (centred / s[..., None]).round().clamp(-127, 127)
        x8, scale = unica.quantize_int8(xd, mean, block)
        assert torch.equal(scale.repeat_interleave(block, -1)[..., :n], s), (shape, block)
        assert torch.equal(unica.decode_int8(x8, n).float(), codes), (shape, block)
        o_codes, o_scales = oracle.quantize_int8(x, None if mean is None else mean.cpu(), block, recip=True)
        assert np.array_equal(np_heads(s[..., ::block]), o_scales) and np.array_equal(np_heads(codes), o_codes)


@pytest.mark.parametrize("shape", SHAPES)
def test_v_scales(shape):
    import unicaattention_b200 as unica

    v = randn_bf16(shape, 12, channel_scale=True)
    vd = v.cuda()
    n = shape[2]
    # per channel: unica/__init__.py:426-427, amax over the tokens / 127.0 on a CUDA tensor
    low, high = torch.aminmax(vd.float(), dim=-2)
    s = (torch.maximum(high, -low) / 127.0).clamp_min(1e-12)
    v8, scale = unica.quantize_v(vd)
    assert torch.equal(scale, s)
    assert torch.equal(unica.decode_v8(v8, n).float(), (vd.float() / s[..., None, :]).round().clamp(-127, 127))
    assert np.array_equal(np_heads(s), oracle.quantize_v_channel(v, recip=True)[1])
    # per token: bench/emulate.py:279-287, amax over the channels / 127.0
    st = (vd.float().abs().amax(-1) / 127.0).clamp_min(1e-12)
    v8, _, tok = unica.quantize_v(vd, per_token=True)
    codes = (vd.float() / st[..., None]).round().clamp(-127, 127)
    assert torch.equal(unica.decode_v8(v8, n).float(), codes)
    inv = tok[:, :, :, 1].flatten(-2)[..., :n]
    assert torch.equal(inv, 1.0 / st)
    o_codes, o_s, _, o_inv = oracle.quantize_v_token(v, recip=True)
    assert np.array_equal(np_heads(st), o_s) and np.array_equal(np_heads(codes), o_codes)


@pytest.mark.parametrize("n", [64, 1000])
def test_nvfp4_scales(n):
    """outer = amax / (6 * 448), scale byte = e4m3(amax16 / 6 / outer): the two divisions by a number are reciprocal
    multiplies on CUDA, the one by the outer tensor a true division."""
    import unicaattention_b200 as unica

    x = randn_bf16((1, 3, n, 128), 13, channel_scale=True)
    xd = x.cuda()
    mean = unica.rope_stats(xd)[0]
    centred = xd.float() - mean[..., None, :]
    blocks = centred.unflatten(-1, (-1, 16))
    amax = blocks.abs().amax(-1, keepdim=True)
    outer = (amax.amax((-3, -2, -1), keepdim=True) / (6.0 * 448.0)).clamp_min(1e-30)
    sf = (amax / 6.0 / outer).clamp(max=448.0).to(torch.float8_e4m3fn)
    k4, k_outer = unica.quantize_fp4_rows(xd, mean, 64)
    _, got_sf = unica.decode_fp4_rows(k4, n, slots=True)
    assert torch.equal(k_outer, outer[..., 0, 0, 0])
    assert torch.equal(got_sf, sf[..., 0].view(torch.uint8))
    _, o_sf, o_outer = oracle.nvfp4_rows(x, mean.cpu(), 0, recip=True)
    assert np.array_equal(np_heads(outer[..., 0, 0]).reshape(-1), o_outer.reshape(-1))
    assert np.array_equal(np_heads(sf[..., 0].view(torch.uint8)), o_sf)
