"""tcgen05.mma kind::i8 on small integers: every result is exact, so a wrong lane, layout or signedness cannot hide
(the idea of the reference's tests/test_mma.py).  Also pins the operand image the quantizers write."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def image(m: np.ndarray) -> np.ndarray:
    """[rows, k] -> [k / 16][rows][16]: the no-swizzle K-major operand image."""
    rows, k = m.shape
    return np.ascontiguousarray(m.reshape(rows, k // 16, 16).transpose(1, 0, 2))


@pytest.mark.parametrize("n,k,unsigned", [(64, 128, False), (128, 64, True), (32, 32, False), (128, 128, True)])
def test_mma_i8_exact(n, k, unsigned):
    from unicaattention_b200 import lib

    rng = np.random.default_rng(n + k)
    a = rng.integers(0, 256, (128, k)).astype(np.uint8) if unsigned else rng.integers(-127, 128, (128, k)).astype(np.int8)
    b = rng.integers(-127, 128, (n, k)).astype(np.int8)
    expected = a.astype(np.int64) @ b.astype(np.int64).T
    a_dev = torch.from_numpy(image(a).view(np.uint8)).cuda()
    b_dev = torch.from_numpy(image(b).view(np.uint8)).cuda()
    d = torch.full((128, n), -1, dtype=torch.int32, device="cuda")
    lib.call("unica_b200_selftest_mma_i8", lib.ptr(a_dev), lib.ptr(b_dev), n, k, int(unsigned), 0, lib.ptr(d), lib.stream())
    got = d.cpu().numpy().astype(np.int64)
    assert np.array_equal(got, expected), f"{np.sum(got != expected)} of {got.size} differ"


@pytest.mark.parametrize("n,k_values", [(64, 32), (32, 8), (128, 16)])
def test_mma_tf32_exact(n, k_values):
    """kind::tf32 as the smoothing-table kernel issues it: small integers, and values that need tf32's 11 bits."""
    from unicaattention_b200 import lib

    rng = np.random.default_rng(n + k_values)
    a = rng.integers(-1023, 1024, (128, k_values)).astype(np.float32)  # 11 significant bits: exact in tf32
    b = (rng.integers(-15, 16, (n, k_values)) / 4.0).astype(np.float32)
    expected = (a.astype(np.float64) @ b.astype(np.float64).T).astype(np.float32)  # sums below 2^24 / 4: exact in float
    a_dev = torch.from_numpy(image(a.view(np.uint8).reshape(128, -1))).cuda()
    b_dev = torch.from_numpy(image(b.view(np.uint8).reshape(n, -1))).cuda()
    d = torch.full((128, n), -1, dtype=torch.int32, device="cuda")
    lib.call("unica_b200_selftest_mma_i8", lib.ptr(a_dev), lib.ptr(b_dev), n, 4 * k_values, 2, 0, lib.ptr(d), lib.stream())
    got = d.cpu().numpy().view(np.float32)
    assert np.array_equal(got, expected), f"{np.sum(got != expected)} of {got.size} differ"


E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)
SCALE_BYTES = np.array([0x30, 0x38, 0x3C, 0x40, 0x44, 0x28], dtype=np.uint8)  # 0.5, 1, 1.5, 2, 3, 0.25 in e4m3


def fp4_image(codes: np.ndarray) -> np.ndarray:
    """4-bit codes [rows, k] -> [k / 32][rows][16] bytes, two codes per byte, the lower k in the low nibble."""
    rows, k = codes.shape
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)  # [rows, k / 2]
    return np.ascontiguousarray(packed.reshape(rows, k // 32, 16).transpose(1, 0, 2))


@pytest.mark.parametrize("n,k,variant", [(64, 128, 0), (144, 64, 0), (128, 64, 0), (16, 64, 0), (64, 128, 2), (144, 64, 2)])
def test_mma_nvf4_exact(n, k, variant):
    from unicaattention_b200 import lib

    rng = np.random.default_rng(n * 7 + k)
    a = rng.integers(0, 16, (128, k)).astype(np.uint8)
    b = rng.integers(0, 16, (n, k)).astype(np.uint8)
    sfa = SCALE_BYTES[rng.integers(0, len(SCALE_BYTES), (128, k // 16))]
    sfb = SCALE_BYTES[rng.integers(0, len(SCALE_BYTES), (n, k // 16))]
    decode = lambda bytes_: torch.from_numpy(np.ascontiguousarray(bytes_)).view(torch.float8_e4m3fn).float().numpy()
    a_val = E2M1[a] * np.repeat(decode(sfa), 16, 1)
    b_val = E2M1[b] * np.repeat(decode(sfb), 16, 1)
    expected = a_val.astype(np.float64) @ b_val.astype(np.float64).T  # every partial sum is exact in float32 too
    words = lambda sf, rows: np.ascontiguousarray(sf.reshape(rows, k // 64, 4).transpose(1, 0, 2)).view(np.uint32)  # [k / 64][rows]
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x).view(np.uint8)).cuda()
    a_dev, b_dev, sfa_dev, sfb_dev = dev(fp4_image(a)), dev(fp4_image(b)), dev(words(sfa, 128)), dev(words(sfb, n))
    d = torch.full((128, n), float("nan"), device="cuda")
    lib.call("unica_b200_selftest_mma_nvf4", lib.ptr(a_dev), lib.ptr(b_dev), lib.ptr(sfa_dev), lib.ptr(sfb_dev), n, k, variant,
             lib.ptr(d), lib.stream())
    got = d.cpu().numpy().astype(np.float64)
    assert np.array_equal(got, expected), f"{np.sum(got != expected)} of {got.size} differ; max {np.abs(got - expected).max()}"
