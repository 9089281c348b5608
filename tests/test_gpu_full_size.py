"""The presets at BASELINE's full shape (1 x 40 x 32760 x 128), where the oracle is far too slow, held to properties that
do not depend on the size: a head's result does not depend on the other heads in the call (bit for bit), doubling V
doubles the output (exactly where the V scale is per channel: the codes do not change and x2 is exact in bf16), a constant V
comes back as that constant, and a sample of rows agrees with the oracle's emulation (one head, a few hundred queries,
all keys)."""

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
HEADS, TOKENS = 40, 32760
MODES = {"per_channel": oracle.V_CHANNEL, "per_token": oracle.V_TOKEN, "outliers": oracle.V_OUTLIERS}


@pytest.fixture(scope="module")
def full():
    g = torch.Generator(device="cuda").manual_seed(2024)
    q, k, v = (torch.randn((1, HEADS, TOKENS, 128), device="cuda", dtype=torch.bfloat16, generator=g) for _ in range(3))
    k += 0.25  # a mean for the K centring to take away
    v[0, :, 1234] *= 50  # a token for the outliers preset and the per-token scales to deal with
    yield q, k, v
    del q, k, v
    torch.cuda.empty_cache()


@pytest.mark.parametrize("preset", ["per_channel", "per_token", "outliers", "fast"])
def test_properties_at_full_size(full, preset):
    import unicaattention_b200 as unica

    q, k, v = full
    settings = unica.PRESETS[preset]
    out = unica.attention(q, k, v, **settings)
    unica.check_status()
    assert out.shape == q.shape and bool(torch.isfinite(out).all())
    # a head alone gives the same bits as inside the full call
    for head in (0, 17, 39):
        alone = unica.attention(q[:, head:head + 1], k[:, head:head + 1], v[:, head:head + 1], **settings)
        assert torch.equal(alone[:, 0], out[:, head]), (preset, head)
    # doubling V doubles the output: exactly where V's scales are per channel (they double, the codes stay); per token the
    # scale enters the scores as log2 s, whose rounding moves with the binade, so only to rounding there
    doubled = unica.attention(q, k, v * 2, **settings)
    if preset == "per_token":
        assert ((doubled.float() - 2 * out.float()).norm() / (2 * out.float()).norm()).item() < 2e-3
    else:
        assert torch.equal(doubled, out * 2), preset
    # a constant V comes back (the weights of a row sum to one)
    five = unica.attention(q[:, :2], k[:, :2], torch.full_like(v[:, :2], 5.0), **settings)
    assert (five.float() - 5.0).abs().max().item() < (0.08 if preset == "fast" else 0.03), (five.float() - 5.0).abs().max().item()
    unica.check_status()


@pytest.mark.parametrize("preset", ["per_channel", "per_token", "outliers", "fast"])
def test_a_sample_of_rows_against_the_emulation(full, preset):
    import unicaattention_b200 as unica

    q, k, v = (x[:, 7:8] for x in full)
    first, count = 20000, 192
    out = unica.attention(q, k, v, **unica.PRESETS[preset])[0, 0, first:first + count].float().cpu().numpy()[None]
    host = [x[0].cpu() for x in (q, k, v)]
    if preset == "fast":
        want = oracle.attention_fast(*host, 512, recip=True, k_mean=unica.rope_stats(k)[0].cpu(), q_mean=unica.rope_stats(q, None, 512)[0].cpu(),
                                     q_first=first, q_count=count)
    else:
        want = oracle.attention_accurate(*host, MODES[preset], recip=True, k_mean=unica.quantize_k(k)[2].cpu(), q_first=first, q_count=count)
    assert oracle.rel_l2(out, want) < 2e-3, (preset, oracle.rel_l2(out, want))
