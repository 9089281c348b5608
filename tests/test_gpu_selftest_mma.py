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
