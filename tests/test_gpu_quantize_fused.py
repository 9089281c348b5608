"""The one-launch quantizers of K and V (statistics and codes in one cooperative kernel) against the separate passes
they replace, which are pinned to the oracle elsewhere."""

import pytest
import torch

pytestmark = pytest.mark.gpu
SHAPES = [(1, 2, 1), (1, 3, 64), (2, 2, 65), (1, 5, 1000), (1, 40, 4097), (1, 70, 300), (1, 2, 20000)]


def tensor(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    batch, heads, n = shape
    x = torch.randn((batch, heads, n, 128), generator=g) * (torch.rand(128, generator=g) * 4) + torch.randn(128, generator=g)
    return x.to(dtype).cuda()


@pytest.mark.parametrize("shape", SHAPES)
def test_v_equals_the_separate_passes(shape):
    import unicaattention_b200 as unica

    v = tensor(shape, 3)
    v8, scale = unica.quantize_v_channel(v)
    want8, want_scale = unica.quantize_v(v)
    unica.check_status()
    assert torch.equal(scale, want_scale) and torch.equal(v8, want8)


@pytest.mark.parametrize("shape", SHAPES)
def test_k_equals_the_separate_passes_on_its_own_mean(shape):
    import unicaattention_b200 as unica

    k = tensor(shape, 5)
    k8, scale, mean = unica.quantize_k(k)
    unica.check_status()
    want8, want_scale = unica.quantize_int8(k, mean, 64)
    assert torch.equal(scale, want_scale) and torch.equal(k8, want8)
    exact = k.double().mean(-2)
    spread = k.double().abs().mean(-2)
    assert ((mean.double() - exact).abs() <= spread * 1e-5 + 1e-7).all()
    other = unica.rope_stats(k)[0]  # the separate pass adds the same terms in another order
    assert ((mean - other).abs() <= spread.float() * 1e-5 + 1e-7).all()


def test_a_head_does_not_depend_on_its_company():
    import unicaattention_b200 as unica

    k = tensor((1, 12, 3000), 7)
    whole = unica.quantize_k(k)
    for piece in (slice(0, 1), slice(3, 8), slice(11, 12)):
        part = unica.quantize_k(k[:, piece])
        assert all(torch.equal(a, b[:, piece]) for a, b in zip(part, whole))
    again = unica.quantize_k(k)
    assert all(torch.equal(a, b) for a, b in zip(again, whole))


def test_float16_and_strided_input():
    import unicaattention_b200 as unica

    k = tensor((1, 3, 900), 9, torch.float16)
    assert all(torch.equal(a, b) for a, b in zip(unica.quantize_k(k), unica.quantize_k(k.bfloat16())))
    v = tensor((1, 3, 900), 10, torch.float16)
    assert all(torch.equal(a, b) for a, b in zip(unica.quantize_v_channel(v), unica.quantize_v_channel(v.bfloat16())))
    nhd = tensor((1, 3, 900), 11).transpose(1, 2).contiguous().transpose(1, 2)  # [batch, tokens, heads, 128] underneath
    assert all(torch.equal(a, b) for a, b in zip(unica.quantize_k(nhd), unica.quantize_k(nhd.contiguous())))


def test_arguments_are_checked():
    import unicaattention_b200 as unica
    from unicaattention_b200 import lib

    k = tensor((1, 1, 128), 1)
    out = torch.empty(1 << 16, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):  # scratch too small
        lib.call("unica_b200_quantize_k_int8_fused", lib.ptr(k), unica.token_layout(k), 1, 128, 2, lib.ptr(out), 1024, lib.ptr(out),
                 lib.ptr(out), lib.ptr(out), None, lib.stream())
    with pytest.raises(ValueError):  # tiles not ceil(n / 64)
        lib.call("unica_b200_quantize_k_int8_fused", lib.ptr(k), unica.token_layout(k), 1, 128, 3, lib.ptr(out), unica.FUSED_SCRATCH_BYTES,
                 lib.ptr(out), lib.ptr(out), lib.ptr(out), None, lib.stream())
