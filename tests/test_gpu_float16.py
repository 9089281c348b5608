"""float16 q, k, v are read in place: every element is rounded to bfloat16 on its way into the statistics and the
quantizers, so the result must be, bit for bit, that of converting the tensors first; where a float16 value is a
bfloat16 value already, that is also the result for the same numbers given as bfloat16."""

import pytest
import torch

pytestmark = pytest.mark.gpu
PRESETS = ["per_channel", "per_token", "outliers", "fast"]


def inputs(heads, n_queries, n_keys, seed, exact=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((1, heads, n_queries, 128), generator=g)
    k, v = (torch.randn((1, heads, n_keys, 128), generator=g) + 0.2 for _ in range(2))
    v[0, :, 5] *= 30
    if exact:  # values both formats hold exactly
        q, k, v = (t.bfloat16().half().float() for t in (q, k, v))
        assert all(torch.equal(t.half().float(), t.bfloat16().float()) for t in (q, k, v))
    return [t.half().cuda() for t in (q, k, v)]


@pytest.mark.parametrize("preset", PRESETS)
@pytest.mark.parametrize("shape", [(3, 700, 700), (2, 130, 1000)])
def test_float16_equals_converting_first(preset, shape):
    import unicaattention_b200 as unica

    q, k, v = inputs(*shape, seed=sum(shape))
    got = unica.attention(q, k, v, **unica.PRESETS[preset])
    want = unica.attention(q.bfloat16(), k.bfloat16(), v.bfloat16(), **unica.PRESETS[preset])
    unica.check_status()
    assert got.dtype == torch.float16 and torch.equal(got, want.half())


@pytest.mark.parametrize("preset", PRESETS)
def test_representable_values_give_the_bfloat16_result(preset):
    import unicaattention_b200 as unica

    q, k, v = inputs(2, 333, 333, seed=4, exact=True)
    got = unica.attention(q, k, v, **unica.PRESETS[preset])
    want = unica.attention(q.float().bfloat16(), k.float().bfloat16(), v.float().bfloat16(), **unica.PRESETS[preset])
    assert torch.equal(got, want.half())


def test_statistics_and_operands_of_float16():
    import unicaattention_b200 as unica

    q, k, v = inputs(2, 515, 515, seed=8)
    for a, b in zip(unica.rope_stats(k), unica.rope_stats(k.bfloat16())):
        assert torch.equal(a, b)
    for a, b in zip(unica.kernel_inputs(q, k, v, **unica.PRESETS["per_channel"])[:6], unica.kernel_inputs(q.bfloat16(), k.bfloat16(), v.bfloat16(), **unica.PRESETS["per_channel"])[:6]):
        assert torch.equal(a, b)


def test_float16_in_the_layout_of_a_sampler():
    """[batch, tokens, heads, 128] float16 through a transposed view, output in the same layout, no copies asked of torch."""
    import unicaattention_b200 as unica

    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn((1, 400, 4, 128), generator=g).half().cuda().transpose(1, 2) for _ in range(3))
    got = unica.attention(q, k, v, **unica.PRESETS["per_channel"])
    assert got.stride() == q.stride() and got.dtype == torch.float16
    want = unica.attention(*(t.contiguous().bfloat16() for t in (q, k, v)), **unica.PRESETS["per_channel"])
    assert torch.equal(got, want.half())
