"""Pins the CPU oracle (oracle/unica_oracle.c) to the reference emulator's own numbers.

tests/golden/golden.npz was produced by tests/golden/make_golden.py from the reference's bench/emulate.py on CPU tensors;
on the CPU torch divides by a scalar exactly, which is the oracle's recip=False form.  Codes and scales must match bit
for bit (hashes of the emulator's arrays); attention outputs must match to float rounding.
"""

import hashlib

import numpy as np
import pytest
import torch

import oracle

CASES = ("cfg1", "ragged", "outlier")


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def inputs(golden, name):
    if name == "cfg1":  # the reference's seed-0 recipe (bench/emulate.py:447-449), regenerated
        torch.manual_seed(0)
        q, k, v = (torch.randn((1, 4, 1024, 128), dtype=torch.bfloat16) for _ in range(3))
        q, k, v = (oracle.bf16_bits(t) for t in (q, k, v))
    else:
        q, k, v = (golden[f"{name}/{t}"].reshape(-1, golden[f"{name}/{t}"].shape[-2], 128) for t in "qkv")
    got = sha(np.concatenate([t.ravel() for t in (q, k, v)]))
    assert got == str(golden[f"{name}/input_sha"]), "the seeded inputs differ from the ones the fixture was made from"
    return q, k, v


def test_e2m1_known_answers(golden):
    lib = oracle.lib()
    decode = lambda xs: np.array([lib.uo_e2m1_to_float(lib.uo_float_to_e2m1(float(x))) for x in xs], np.float32)
    assert np.array_equal(decode(golden["e2m1/grid"]), golden["e2m1/grid"])
    assert np.array_equal(decode(golden["e2m1/ties_in"]), golden["e2m1/ties_out"])  # [0,1,1,2,2,4,4]
    assert np.array_equal(decode(golden["e2m1/sat_in"]), golden["e2m1/sat_out"])  # [6,6,-6]
    assert np.array_equal(decode(golden["e2m1/sweep_in"]), golden["e2m1/sweep_out"])


def test_e4m3_matches_torch(golden):
    lib = oracle.lib()
    got = np.array([lib.uo_float_to_e4m3(float(x)) for x in golden["e4m3/in"]], np.uint8)
    assert np.array_equal(got, golden["e4m3/bytes"])
    every = np.arange(127, dtype=np.uint8)  # every finite non-negative e4m3 value decodes as torch decodes it
    expected = torch.from_numpy(every).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.array([lib.uo_e4m3_to_float(int(b)) for b in every], np.float32), expected)


def test_slot_order(golden):
    assert np.array_equal(oracle.slot_key(), golden["slot_key"])


@pytest.mark.parametrize("name", CASES)
def test_int8_quantizers_bit_exact(golden, name):
    q, k, v = inputs(golden, name)
    g = lambda key: golden[f"{name}/{key}"]
    heads = q.shape[0]
    q8, sq = oracle.quantize_int8(q, None, 128, recip=False)
    k8, sk = oracle.quantize_int8(k, g("k_mean").reshape(heads, 128), 64, recip=False)
    assert np.array_equal(sq, g("q_scale").reshape(sq.shape)) and sha(q8) == str(g("q8_sha"))
    assert np.array_equal(sk, g("k_scale").reshape(sk.shape)) and sha(k8) == str(g("k8_sha"))
    v8, sv = oracle.quantize_v_channel(v, recip=False)
    assert np.array_equal(sv, g("v_scale").reshape(sv.shape)) and sha(v8) == str(g("v8_sha"))
    v8t, s_tok, _, _ = oracle.quantize_v_token(v, recip=False)
    assert np.array_equal(s_tok, g("v_tok_scale").reshape(s_tok.shape)) and sha(v8t) == str(g("v8t_sha"))


def dequant_rows(codes, sf, outer):
    scales = torch.from_numpy(sf).view(torch.float8_e4m3fn).float().numpy() * outer[:, None, None]
    return oracle.E2M1_VALUES[codes] * np.repeat(scales, 16, -1)


@pytest.mark.parametrize("name", CASES)
def test_nvfp4_quantizers_bit_exact(golden, name):
    q, k, v = inputs(golden, name)
    g = lambda key: golden[f"{name}/{key}"]
    heads = q.shape[0]
    qc, qsf, qo = oracle.nvfp4_rows(q, g("q_mean").reshape(heads, -1, 128), 512, recip=False)
    kc, ksf, ko = oracle.nvfp4_rows(k, g("k_mean").reshape(heads, 1, 128), 0, recip=False)
    assert np.array_equal(qo, g("q4_outer").reshape(qo.shape)) and np.array_equal(ko, g("k4_outer").reshape(ko.shape))
    assert sha(qsf) == str(g("q4_sf_sha")) and sha(ksf) == str(g("k4_sf_sha"))
    assert sha(dequant_rows(qc, qsf, qo)) == str(g("q4_deq_sha"))
    assert sha(dequant_rows(kc, ksf, ko)) == str(g("k4_deq_sha"))
    vc, vsf, vo = oracle.nvfp4_v(v, recip=False)
    assert np.array_equal(vo, g("v4_outer").reshape(vo.shape))
    # emulator: blocks along keys, [heads, 128, tiles * 4] scale bytes; ours: [heads, tiles, 4, 128]
    tiles = vsf.shape[1]
    assert sha(np.ascontiguousarray(vsf.reshape(heads, tiles * 4, 128).transpose(0, 2, 1))) == str(g("v4_sf_sha"))
    scales = torch.from_numpy(vsf).view(torch.float8_e4m3fn).float().numpy() * vo[:, None, None, :]
    deq = oracle.E2M1_VALUES[vc] * np.repeat(scales, 16, 2).reshape(heads, tiles * 64, 128)
    assert sha(deq) == str(g("v4_deq_sha"))


def rows_of(golden, name, nq):
    n_rows = {"cfg1": 64, "ragged": None, "outlier": 128}[name]
    return slice(None) if n_rows is None else slice(0, None, max(1, nq // n_rows))


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("mode", ["per_channel", "per_token", "outliers", "fast", "fast_unsmoothed"])
def test_attention_matches_emulator(golden, name, mode):
    q, k, v = inputs(golden, name)
    g = lambda key: golden[f"{name}/{key}"]
    heads, nq, _ = q.shape
    k_mean = g("k_mean").reshape(heads, 128)  # torch's own k.mean, so that both sides quantize the same centred K
    if mode.startswith("fast"):
        smooth = 512 if mode == "fast" else 0
        out = oracle.attention_fast(q, k, v, smooth, recip=False, k_mean=k_mean,
                                    q_mean=g("q_mean").reshape(heads, -1, 128) if smooth else None)
    else:
        v_mode = {"per_channel": oracle.V_CHANNEL, "per_token": oracle.V_TOKEN, "outliers": oracle.V_OUTLIERS}[mode]
        out = oracle.attention_accurate(q, k, v, v_mode, 8, recip=False, k_mean=k_mean)
    sel = rows_of(golden, name, nq)
    expected = oracle.bf16_to_float(g(f"out_{mode}").reshape(heads, -1, 128))
    got = out[:, sel]
    # same integers in, float sums in another order: a few outputs land on the neighbouring bf16 value
    assert oracle.rel_l2(got, expected) < 2e-4, oracle.rel_l2(got, expected)
    assert np.mean(got != expected) < 0.02
    # and the error against FP32 is the emulator's
    err = oracle.rel_l2(got, g("ref").reshape(heads, -1, 128))
    full = oracle.rel_l2(out, oracle.reference_fp32(q, k, v))
    assert abs(full - float(g(f"err_{mode}"))) < 2e-4 * max(1.0, float(g(f"err_{mode}")) / 0.02), (full, float(g(f"err_{mode}")), err)


def test_own_statistics_agree_with_torch(golden):
    """The fixed-order means of the oracle are the 1e-6 neighbours of torch's (tests/test_rope.py:43 in the reference)."""
    q, k, v = inputs(golden, "outlier")
    mean, low, high = oracle.channel_stats(k)
    kf = oracle.bf16_to_float(k)
    assert np.allclose(mean[:, 0], golden["outlier/k_mean"].reshape(-1, 128), atol=1e-6)
    assert np.array_equal(low[:, 0], kf.min(1)) and np.array_equal(high[:, 0], kf.max(1))
    qm, _, _ = oracle.channel_stats(q, 512)
    assert np.allclose(qm, golden["outlier/q_mean"].reshape(qm.shape), atol=1e-5)
