"""Pins the oracle's RoPE path to the reference emulator: tests/golden/golden_rope.npz holds what bench/emulate.py gives
on inputs rotated by its rope() (made by tests/golden/make_golden_rope.py on CPU tensors, so scalar divisions are IEEE
divisions: the oracle's recip=False form).  The case is the reference's own (tests/test_rope.py:24-35)."""

import hashlib

import numpy as np
import pytest

import oracle

T, H, W = 3, 7, 9


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def inputs(g):
    return g["q"].reshape(-1, T * H * W, 128), g["k"].reshape(-1, T * H * W, 128), g["v"].reshape(-1, T * H * W, 128)


def test_the_table_builder_is_the_emulators(golden_rope):
    assert np.array_equal(oracle.wan_rope_table(T, H, W), golden_rope["table"])


def test_rotation_bit_exact(golden_rope):
    q, k, _ = inputs(golden_rope)
    table = golden_rope["table"]
    assert sha(oracle.rope_rotate(q, table)) == str(golden_rope["q_rot_sha"])
    assert sha(oracle.rope_rotate(k, table)) == str(golden_rope["k_rot_sha"])


def test_statistics_and_quantizers_of_the_rotated_tensors(golden_rope):
    g = golden_rope
    q, k, _ = inputs(g)
    table = g["table"]
    mean, low, high = oracle.channel_stats(k, 0, rope=table)
    assert np.array_equal(low[:, 0], g["k_low"][0]) and np.array_equal(high[:, 0], g["k_high"][0])
    assert np.allclose(mean[:, 0], g["k_mean"][0], rtol=0, atol=1e-6)  # the reference's own tolerance (tests/test_rope.py:43)
    k8, k_scale = oracle.quantize_int8(k, g["k_mean"][0], 64, recip=False, rope=table)
    assert sha(k8) == str(g["k8_sha"]) and np.array_equal(k_scale, g["k_scale"][0])
    q8, q_scale = oracle.quantize_int8(q, None, 128, recip=False, rope=table)
    assert sha(q8) == str(g["q8_sha"]) and np.array_equal(q_scale, g["q_scale"][0])
    codes, sf, outer = oracle.nvfp4_rows(q, recip=False, rope=table)
    e4m3 = np.array([oracle.lib().uo_e4m3_to_float(b) for b in range(256)], np.float32)
    deq = np.array(oracle.E2M1_VALUES, np.float32)[codes] * np.repeat(e4m3[sf] * outer[:, None, None], 16, -1)
    assert sha(deq.reshape(1, *deq.shape)) == str(g["q4_deq_sha"])


@pytest.mark.parametrize("mode", ["per_channel", "per_token", "fast", "fast_unsmoothed"])
def test_attention_on_rotated_inputs(golden_rope, mode):
    g = golden_rope
    q, k, v = inputs(g)
    table = g["table"]
    if mode.startswith("fast"):
        got = oracle.attention_fast(q, k, v, 256 if mode == "fast" else 0, recip=False, k_mean=g["k_mean"][0], rope=table)
    else:
        v_mode = {"per_channel": oracle.V_CHANNEL, "per_token": oracle.V_TOKEN}[mode]
        got = oracle.attention_accurate(q, k, v, v_mode, recip=False, k_mean=g["k_mean"][0], rope=table)
    want = oracle.bf16_to_float(g["out_" + mode].reshape(got.shape))
    ref = oracle.reference_fp32(q, k, v, rope=table)
    assert oracle.rel_l2(ref, g["ref"].reshape(ref.shape)) < 1e-5
    assert oracle.rel_l2(got, want) < (2e-3 if mode.startswith("fast") else 3e-4), oracle.rel_l2(got, want)
    assert abs(oracle.rel_l2(got, ref) - float(g["err_" + mode])) < 0.02 * float(g["err_" + mode]) + 1e-4
