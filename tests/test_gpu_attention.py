"""The accurate-mode attention kernel against the oracle, through the public call and the C ABI underneath.

Gates (tolerances from the task's contract): output within rel-L2 2e-3 of the emulation (the reference's own test
limit is 1e-3, tests/test_attention.py:33); error against FP32 no worse than the emulation's + 1e-4 (its
tests/test_fp4.py:90 idiom)."""

import numpy as np
import pytest
import torch

import oracle
from gpu_common import EDGE_SHAPES, out_heads, qkv, rel_l2

pytestmark = pytest.mark.gpu
FROM_EMULATION = 2e-3
MODES = {"per_channel": oracle.V_CHANNEL, "per_token": oracle.V_TOKEN, "outliers": oracle.V_OUTLIERS}


def run(q, k, v, preset):
    import unicaattention_b200 as unica

    out = unica.attention(q.cuda(), k.cuda(), v.cuda(), **unica.PRESETS[preset])
    unica.check_status()
    k_mean = unica.quantize_k(k.cuda())[2].cpu()  # the mean the call itself took away
    return out, k_mean


@pytest.mark.parametrize("preset", list(MODES))
@pytest.mark.parametrize("shape", EDGE_SHAPES)
def test_matches_emulation_on_edge_shapes(shape, preset):
    batch, heads, nq, nk = shape
    q, k, v = qkv(batch, heads, nq, nk, seed=nq + nk)
    out, k_mean = run(q, k, v, preset)
    assert out.shape == q.shape and out.dtype == q.dtype and torch.isfinite(out).all()
    got = out_heads(out)
    want = oracle.attention_accurate(q, k, v, MODES[preset], recip=True, k_mean=k_mean)
    assert rel_l2(got, want) < FROM_EMULATION, (shape, preset, rel_l2(got, want))
    ref = oracle.reference_fp32(q, k, v)
    assert rel_l2(got, ref) <= rel_l2(want, ref) + 1e-4


@pytest.mark.parametrize("preset", list(MODES))
def test_repeats_are_bit_identical(preset):
    """Three runs: a race between the pipeline's stages would show as a difference (tests/test_attention.py:205)."""
    import unicaattention_b200 as unica

    q, k, v = (t.cuda() for t in qkv(1, 3, 777, 1300, seed=11))
    first = unica.attention(q, k, v, **unica.PRESETS[preset])
    for _ in range(2):
        assert torch.equal(unica.attention(q, k, v, **unica.PRESETS[preset]), first)
    unica.check_status()


def test_config1_against_the_reference_emulator_itself(golden):
    """BASELINE config 1 (seed 0, 1x4x1024x128): the kernel against outputs the reference's emulator produced."""
    torch.manual_seed(0)
    q, k, v = (torch.randn((1, 4, 1024, 128), dtype=torch.bfloat16) for _ in range(3))
    ref = golden["cfg1/ref"].reshape(4, -1, 128)
    step = 1024 // 64
    for preset in MODES:
        out, _ = run(q, k, v, preset)
        got = out_heads(out)[:, ::step]
        want = oracle.bf16_to_float(golden[f"cfg1/out_{preset}"].reshape(4, -1, 128))
        assert rel_l2(got, want) < FROM_EMULATION, (preset, rel_l2(got, want))
        assert rel_l2(got, ref) <= float(golden[f"cfg1/err_{preset}"]) * 1.05 + 1e-4


def test_outlier_tokens_need_the_per_token_scale(golden):
    """V tokens 65x and 250x the rest: per channel loses its steps to them, per token does not (tests/test_v_token.py:44-59)."""
    q, k, v = (torch.from_numpy(golden[f"outlier/{t}"].view(np.int16)).view(torch.bfloat16) for t in "qkv")
    ref = oracle.reference_fp32(q, k, v)
    errors = {}
    for preset in MODES:
        out, k_mean = run(q, k, v, preset)
        want = oracle.attention_accurate(q, k, v, MODES[preset], recip=True, k_mean=k_mean)
        assert rel_l2(out_heads(out), want) < FROM_EMULATION
        errors[preset] = rel_l2(out_heads(out), ref)
    assert errors["per_token"] < errors["per_channel"] / 2
    assert errors["outliers"] < errors["per_channel"] / 2  # tests/test_v_outliers.py: the exact add-back does as well


def test_layout_dtype_and_pieces():
    """Output keeps the caller's strides; float16 goes through bf16 pieces; head-split == one call, bit for bit
    (tests/test_pieces.py:17-43, tests/test_attention.py:273-284)."""
    import unicaattention_b200 as unica

    q, k, v = (t.cuda() for t in qkv(2, 4, 700, 700, seed=3))
    whole = unica.attention(q, k, v)
    nhd = [t.transpose(1, 2).contiguous().transpose(1, 2) for t in (q, k, v)]
    strided = unica.attention(*nhd)
    assert strided.stride() == nhd[0].stride() and torch.equal(strided, whole)
    old = unica.heads_per_call
    try:
        unica.heads_per_call = lambda *a, **kw: 3  # 3 + 1 heads
        assert torch.equal(unica.attention(q, k, v), whole)
    finally:
        unica.heads_per_call = old
    half = unica.attention(q.half(), k.half(), v.half())
    assert half.dtype == torch.float16
    assert torch.equal(half, unica.attention(q.half().bfloat16(), k.half().bfloat16(), v.half().bfloat16()).half())
    unica.check_status()


def test_rejects_what_the_kernel_cannot_take():
    import unicaattention_b200 as unica

    q = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        unica.attention(q, q, q)  # head_dim 64
    x = torch.zeros(1, 1, 64, 128, device="cuda")
    with pytest.raises(TypeError):
        unica.attention(x, x, x)  # float32
    b = x.bfloat16()
    with pytest.raises(ValueError):
        unica.attention(b, b[:, :, :0], b[:, :, :0])
    with pytest.raises(ValueError):
        unica.attention(b, b, b, kernel="nope")
    with pytest.raises(ValueError):
        unica.attention(b, b, b, NOPE=1)
    with pytest.raises(ValueError):
        unica.attention(b.cpu(), b.cpu(), b.cpu())


@pytest.mark.parametrize("preset", ["per_channel", "fast"])
def test_host_memory_call_is_the_device_call(preset):
    """attention_host sends the heads through the GPU in groups with the copies overlapping the kernels: bit for bit the
    result of one call on the whole tensors, for pinned and for pageable host memory."""
    import unicaattention_b200 as unica

    q, k, v = qkv(1, 7, 600, 600, seed=5)
    whole = unica.attention(q.cuda(), k.cuda(), v.cuda(), **unica.PRESETS[preset]).cpu()
    pinned = [x.pin_memory() for x in (q, k, v)]
    out = unica.attention_host(*pinned, heads_per_group=3, **unica.PRESETS[preset])
    torch.cuda.synchronize()
    assert out.is_pinned() and torch.equal(out, whole)
    again = torch.empty_like(out)
    assert unica.attention_host(q, k, v, out=again, **unica.PRESETS[preset]) is again
    torch.cuda.synchronize()
    assert torch.equal(again, whole)
    unica.check_status()
    with pytest.raises(ValueError):
        unica.attention_host(q.cuda(), k.cuda(), v.cuda())
