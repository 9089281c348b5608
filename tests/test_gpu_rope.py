"""RoPE inside the quantizers, against the oracle on rotated inputs (the reference's tests/test_rope.py):

1. rope_stats gives each channel's min, max and mean of the rotated x;
2. quantize_int8 and quantize_fp4_rows with rope= are, bit for bit, the quantization of rope(x) - mean;
3. attention(q, k, v, rope=table) is the emulation on the rotated q and k, for every preset, one table for the batch
   or one per batch item;
4. the compact table is kept while the same table comes back, also under torch.inference_mode."""

import numpy as np
import pytest
import torch

import oracle
from gpu_common import np_heads, out_heads, rel_l2

pytestmark = pytest.mark.gpu
T, H, W = 3, 7, 9  # a small latent of WAN's shape: 189 tokens, past a tile edge and a statistics block
FROM_EMULATION = 2e-3


def inputs(heads=3, batch=1, seed=0, latent=(T, H, W)):
    """q, k, v in ComfyUI's layout ([batch, tokens, heads, 128], read through a transpose) and the table."""
    g = torch.Generator().manual_seed(seed)
    tokens = latent[0] * latent[1] * latent[2]
    q, k, v = (torch.randn((batch, tokens, heads, 128), generator=g).bfloat16().transpose(1, 2) for _ in range(3))
    return q, k, v, torch.from_numpy(oracle.wan_rope_table(*latent))


def test_rope_stats():
    import unicaattention_b200 as unica

    q, _, _, table = inputs()
    mean, low, high = unica.rope_stats(q.cuda(), table.cuda())
    o_mean, o_low, o_high = oracle.channel_stats(q, 0, rope=table)
    rotated = oracle.rope_rotate(q, table)
    assert np.array_equal(np_heads(low), rotated.min(1)) and np.array_equal(np_heads(high), rotated.max(1))
    assert np.array_equal(np_heads(mean), o_mean[:, 0])  # the same fixed order
    assert np.allclose(np_heads(mean), rotated.mean(1, dtype=np.float64), atol=1e-6)
    mean, low, high = unica.rope_stats(q.cuda(), table.cuda(), 256)
    for got, want in zip((mean, low, high), oracle.channel_stats(q, 256, rope=table)):
        assert np.array_equal(got.cpu().numpy().reshape(want.shape), want)


def test_quantizers_rotate_like_the_emulation():
    import unicaattention_b200 as unica

    q, k, _, table = inputs()
    qd, kd, td = q.cuda(), k.cuda(), table.cuda()
    n = q.shape[2]
    mean = unica.rope_stats(kd, td)[0]
    k8, k_scale = unica.quantize_int8(kd, mean, unica.K_SCALE_BLOCK, td)
    codes, scales = oracle.quantize_int8(k, mean.cpu(), 64, recip=True, rope=table)
    assert np.array_equal(np_heads(unica.decode_int8(k8, n)), codes), "int8 codes"
    assert np.array_equal(np_heads(k_scale), scales), "int8 scales"
    _, low, high = unica.rope_stats(qd, td)
    q4, outer = unica.quantize_fp4_rows(qd, None, 1, td, (low, high))
    got_codes, got_sf = (np_heads(t) for t in unica.decode_fp4_rows(q4, n))
    o_codes, o_sf, o_outer = oracle.nvfp4_rows(q, None, 0, recip=True, rope=table)
    assert np.array_equal(np_heads(outer[..., None])[:, 0], o_outer) and np.array_equal(got_sf, o_sf)
    live = np.repeat(o_sf, 16, -1) != 0
    assert np.array_equal(got_codes[live], o_codes[live]), "fp4 codes"
    # K in slot order with its mean, the smoothing term from the rotated k
    k4, k_outer = unica.quantize_fp4_rows(kd, mean, 64, td)
    got_codes, got_sf = (np_heads(t) for t in unica.decode_fp4_rows(k4, n, slots=True))
    o_codes, o_sf, o_outer = oracle.nvfp4_rows(k, mean.cpu(), 0, recip=True, rope=table)
    assert np.array_equal(np_heads(k_outer[..., None])[:, 0], o_outer) and np.array_equal(got_sf, o_sf)
    q_mean = unica.rope_stats(qd, td, 256)[0]
    bias = unica.smooth_bias(kd, mean, q_mean, rope=td).cpu().numpy().reshape(3, -1, 192)
    centred = oracle.rope_rotate(k, table) - mean.cpu().numpy().reshape(3, 1, 128)
    want = np.einsum("hbc,hkc->hbk", q_mean.cpu().numpy().reshape(3, -1, 128).astype(np.float64), centred.astype(np.float64))
    key_of = np.array([64 * (s // 64) + unica.fp4.SLOT_KEY[s % 64] for s in range(192)])
    valid = key_of < n
    assert np.allclose(bias[:, :, valid], want[:, :, key_of[valid]] * (128**-0.5 * 1.4426950408889634), rtol=1e-5, atol=1e-4)
    assert np.all(np.isneginf(bias[:, :, ~valid]))  # slots past the last key: -inf keeps them out of the softmax


@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("preset", ["per_channel", "per_token", "outliers", "fast"])
def test_attention_with_rope_is_the_emulation(preset, batch):
    import unicaattention_b200 as unica

    q, k, v, table = inputs(batch=batch, seed=batch)
    if batch == 2:  # a table per batch item: the second one that of the latent read backwards
        table = torch.cat([table, table.flip(1)])
    settings = unica.PRESETS[preset] | (dict(SMOOTH_Q=256) if preset == "fast" else {})
    out = unica.attention(q.cuda(), k.cuda(), v.cuda(), rope=table.cuda(), **settings)
    unica.check_status()
    assert out.stride() == q.stride()
    k_mean = unica.rope_stats(k.cuda(), table.cuda())[0].cpu()
    if preset == "fast":
        q_mean = unica.rope_stats(q.cuda(), table.cuda(), 256)[0].cpu()
        want = oracle.attention_fast(q, k, v, 256, recip=True, k_mean=k_mean, q_mean=q_mean, rope=table)
    else:
        v_mode = {"per_channel": oracle.V_CHANNEL, "per_token": oracle.V_TOKEN, "outliers": oracle.V_OUTLIERS}[preset]
        want = oracle.attention_accurate(q, k, v, v_mode, recip=True, k_mean=k_mean, rope=table)
    got = out_heads(out)
    ref = oracle.reference_fp32(q, k, v, rope=table)
    assert rel_l2(got, want) < (1e-2 if preset == "fast" else FROM_EMULATION), (preset, batch, rel_l2(got, want))
    assert rel_l2(got, ref) <= rel_l2(want, ref) * 1.02 + 1e-4


def test_against_the_reference_emulator_itself(golden_rope):
    """The reference's case (seed 0, 3 heads, 189 tokens): outputs its emulator gave on the rotated q and k."""
    import unicaattention_b200 as unica

    g = golden_rope
    q, k, v = (torch.from_numpy(g[t].view(np.int16)).view(torch.bfloat16).cuda() for t in "qkv")
    table = torch.from_numpy(g["table"]).cuda()
    for preset, settings in (("per_channel", {}), ("per_token", {}), ("fast", dict(SMOOTH_Q=256))):
        out = unica.attention(q, k, v, rope=table, **(unica.PRESETS[preset] | settings))
        want = oracle.bf16_to_float(g["out_" + preset].reshape(3, -1, 128))
        assert rel_l2(out_heads(out), want) < (1e-2 if preset == "fast" else FROM_EMULATION), preset
        assert rel_l2(out_heads(out), g["ref"].reshape(3, -1, 128)) <= float(g["err_" + preset]) * 1.05 + 1e-4


def test_table_checks_and_cache():
    import unicaattention_b200 as unica

    q, k, v, table = inputs()
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    with pytest.raises(ValueError):
        unica.attention(qd, kd[:, :, :100], vd[:, :, :100], rope=table[:, :100].cuda())  # cross-attention
    with pytest.raises(ValueError):
        unica.attention(qd, kd, vd, rope=table[:, :100].cuda())  # too short
    with pytest.raises(ValueError):
        unica.attention(qd, kd, vd, rope=table.cuda().half())
    with pytest.raises(ValueError):
        unica.attention(qd, kd, vd, rope=(table * 2).abs().cuda())  # not rotations
    with torch.inference_mode():  # no version counter there: the weak reference alone tells a new table
        td = torch.from_numpy(oracle.wan_rope_table(T, H, W)).cuda()
        first = unica.attention(qd, kd, vd, rope=td)
        kept = unica.compact_rope(td)
        assert unica.attention(qd, kd, vd, rope=td).equal(first) and unica.compact_rope(td) is kept
    changed = table.cuda()
    a = unica.compact_rope(changed)
    changed[:, 0] = changed[:, 1]
    assert unica.compact_rope(changed) is not a  # modified in place: converted again
