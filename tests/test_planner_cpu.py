"""The head planner's arithmetic (the reference's heads_per_call, unica/__init__.py:208-232) with the driver's answers
replaced: no GPU needed."""

import torch

import unicaattention_b200 as unica

GiB = 2**30


def plan(monkeypatch, free, reserve, shape=(1, 40, 32760, 128), dtype=torch.bfloat16, kernel=unica.DEFAULT_KERNEL, **tile):
    monkeypatch.setattr(unica, "free_vram", lambda device, fresh=False: free)
    monkeypatch.setattr(unica, "vram_reserve", lambda device: reserve)
    q = torch.empty(shape, dtype=dtype, device="meta")
    return unica.heads_per_call(q, q, kernel, tile)


def test_small_calls_run_whole(monkeypatch):
    # 40 heads x 32760 tokens: 25 MB of temporaries per head, 1 GB in all: within a quarter of an 18 GiB reserve
    assert plan(monkeypatch, free=150 * GiB, reserve=18 * GiB) == 40
    assert plan(monkeypatch, free=2 * GiB, reserve=18 * GiB) == 40  # and it fits the free memory


def test_large_calls_are_split_to_stay_above_the_reserve(monkeypatch):
    per_head = 128 * 3 * 118320 * 2  # hires shape, bf16
    free, reserve = 6 * GiB, 4 * GiB
    assert 40 * per_head > reserve // unica.SMALL_CALL_FRACTION
    assert plan(monkeypatch, free, reserve, shape=(1, 40, 118320, 128)) == (free - reserve) // per_head
    assert plan(monkeypatch, free=reserve, reserve=reserve, shape=(1, 40, 118320, 128)) == 1  # never less than a head


def test_float16_costs_the_same_and_the_smoothing_table_more(monkeypatch):
    free, reserve = 6 * GiB, 4 * GiB
    shape = (1, 40, 118320, 128)
    bf16 = plan(monkeypatch, free, reserve, shape)
    assert plan(monkeypatch, free, reserve, shape, dtype=torch.float16) == bf16  # read in place: no bf16 copies
    table = 4 * -(-118320 // 512) * 118320  # one float per key and block of 512 queries
    fast = plan(monkeypatch, free, reserve, shape, kernel="attention_fp4", SMOOTH_Q=512)
    assert fast == (free - reserve) // (128 * 3 * 118320 * 2 + table) < bf16
    assert plan(monkeypatch, free, reserve, shape, kernel="attention_fp4", SMOOTH_Q=0) == bf16


def test_free_vram_is_asked_seldom(monkeypatch):
    calls = []
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device: (calls.append(device), (5 * GiB, 8 * GiB))[1])
    unica._FREE_VRAM.clear()
    assert unica.free_vram("gpu") == 5 * GiB and unica.free_vram("gpu") == 5 * GiB and len(calls) == 1
    monkeypatch.setattr(unica, "FREE_VRAM_MAX_AGE", -1.0)
    assert unica.free_vram("gpu") == 5 * GiB and len(calls) == 2
    unica._FREE_VRAM.clear()


def test_a_large_call_asks_the_driver_again(monkeypatch):
    """A call that needs more than an eighth of the remembered free memory does not trust the remembered figure."""
    answers = iter([(24 * GiB, 180 * GiB), (5 * GiB, 180 * GiB)])
    calls = []
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device: (calls.append(device), next(answers))[1])
    monkeypatch.setattr(unica, "vram_reserve", lambda device: 4 * GiB)
    unica._FREE_VRAM.clear()

    small = torch.empty((1, 2, 1024, 128), dtype=torch.bfloat16, device="meta")
    assert unica.heads_per_call(small, small, unica.DEFAULT_KERNEL, {}) == 2 and len(calls) == 1  # the remembered figure will do
    big = torch.empty((1, 40, 118320, 128), dtype=torch.bfloat16, device="meta")
    per_head = 128 * 3 * 118320 * 2
    assert 40 * per_head > 24 * GiB // unica.STALE_FRACTION
    assert unica.heads_per_call(big, big, unica.DEFAULT_KERNEL, {}) == (5 * GiB - 4 * GiB) // per_head and len(calls) == 2
    unica._FREE_VRAM.clear()
