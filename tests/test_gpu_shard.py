"""The head-sharded call on one GPU (a process group of one rank): the rank's heads go through the kernel in groups whose
outputs are gathered on a side stream, and the result must be bit for bit that of one plain call (every head has its own
statistics and scales).  The two-rank arithmetic of the gather itself is covered on the CPU (tests/test_shard_cpu.py)."""

import socket

import pytest
import torch
import torch.distributed as dist

from gpu_common import qkv

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def one_rank_group():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    yield
    dist.destroy_process_group()


@pytest.mark.parametrize("preset", ["per_channel", "per_token", "outliers", "fast"])
def test_grouped_gather_equals_one_call(one_rank_group, preset):
    import unicaattention_b200 as unica
    from unicaattention_b200 import shard

    q, k, v = (x.cuda() for x in qkv(1, 7, 700, 700, seed=3))
    whole = unica.attention(q, k, v, **unica.PRESETS[preset])
    for groups in (None, 3, 1):
        got = shard.attention_sharded(q, k, v, 7, head_groups=groups, **unica.PRESETS[preset])
        torch.cuda.synchronize()
        assert torch.equal(got, whole), (preset, groups)
    out = torch.empty_like(whole)
    assert shard.attention_sharded(q, k, v, 7, out=out, **unica.PRESETS[preset]) is out
    torch.cuda.synchronize()
    assert torch.equal(out, whole)
    unica.check_status()


def test_slice_heads_keeps_the_operands_types():
    import unicaattention_b200 as unica
    from unicaattention_b200 import shard

    q, k, v = (x.cuda() for x in qkv(1, 4, 300, 300, seed=4))
    inputs = unica.kernel_inputs(q, k, v, **unica.PRESETS["fast"])
    part = shard.slice_heads(inputs, slice(1, 3))
    assert type(part[0]) is type(inputs[0]) and part[0].codes.shape[1] == 2 and part[3].shape == (1, 2)
    assert part[-1] == inputs[-1]  # SMOOTH_Q, a number
    inputs = unica.kernel_inputs(q, k, v, **unica.PRESETS["outliers"])
    keys, rows = shard.slice_heads(inputs, slice(0, 1))[6]
    assert keys.shape[1] == 1 and rows.shape[1] == 1


def test_shared_output_in_a_group_of_one(one_rank_group):
    """SharedOutput and its two barriers with a one-rank group: no peers, the same bits as a plain call."""
    import unicaattention_b200 as unica
    from unicaattention_b200 import shard

    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn((1, 4, 700, 128), device="cuda", dtype=torch.bfloat16, generator=g) for _ in range(3))
    try:
        shared = shard.SharedOutput(1, 4, 700)
    except RuntimeError as error:
        pytest.skip(f"symmetric memory unavailable: {error}")
    for preset in ("per_channel", "fast"):
        got = shard.attention_sharded(q, k, v, 4, out=shared, **unica.PRESETS[preset])
        assert got is shared.tensor and torch.equal(got, unica.attention(q, k, v, **unica.PRESETS[preset]))
    unica.check_status()
