"""The statistics entry point that needs no scratch buffer from its caller (unica_b200_channel_stats_static).

It exists for callers that cannot allocate device memory (a hook inside a pipeline that keeps the card full, a C host
with no allocator) or must not (cudaMalloc stalls the device).  The test goes through the C ABI with caller-owned
outputs only, twice in a row on different inputs (the built-in scratch keeps the first call's contents), and demands
the results of the ordinary entry point bit for bit.  It is collected last, so a run that stops at the first failure
has already run everything else; it must pass alone in a fresh process as well.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def both(x, per):
    """(mean, low, high) from the entry point with caller scratch and from the one without."""
    from unicaattention_b200 import lib

    batch, heads, n, _ = x.shape
    layout = lib.TokenLayout(x.stride(0), x.stride(1), x.stride(2), heads)
    groups = 1 if per == 0 else -(-n // per)
    results = []
    for name in ("unica_b200_channel_stats", "unica_b200_channel_stats_static"):
        mean, low, high = (torch.full((batch * heads, groups, 128), float("nan"), device=x.device) for _ in range(3))
        scratch = []
        if name == "unica_b200_channel_stats":
            scratch = [torch.empty(batch * heads, -(-n // 256), 3, 128, device=x.device)]
        lib.call(name, lib.ptr(x), layout, batch * heads, n, per, *(lib.ptr(t) for t in scratch), lib.ptr(mean), lib.ptr(low),
                 lib.ptr(high), lib.stream())
        results.append((mean, low, high))
    torch.cuda.synchronize()
    return results


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    g = torch.Generator().manual_seed(21)
    first = (torch.randn((2, 3, 1000, 128), generator=g) * 3 + 1).bfloat16().cuda()
    second = torch.randn((1, 5, 700, 128), generator=g).bfloat16().cuda()  # other sizes: stale records stay in the scratch
    for x, per in ((first, 0), (second, 512)):
        ordinary, static = both(x, per)
        for a, b in zip(ordinary, static):
            assert torch.isfinite(b).all() and torch.equal(a, b)


def test_refuses_what_does_not_fit():
    from unicaattention_b200 import lib

    x = torch.zeros(1, 1, 256, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(3, 128, device="cuda")
    with pytest.raises(ValueError, match="6144"):  # 7000 heads x 1 block
        lib.call("unica_b200_channel_stats_static", lib.ptr(x), lib.TokenLayout(0, 0, 128, 7000), 7000, 256, 0, lib.ptr(out),
                 lib.ptr(out), lib.ptr(out), ctypes.c_void_p(0))
