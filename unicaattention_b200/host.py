"""attention() for tensors that live in host memory: the heads go through the GPU in groups (growing at first, a small
one last: see group_sizes), so that the copy of the next group's q, k, v, the kernels of this one and the copy of the previous
group's output run at the same time (three streams).  Heads are independent (every head has its own statistics and scales), so the result is bit for bit that of
one call on the whole tensors.

The reference has no such call: its callers hold their tensors on the GPU.  It is here for hosts that do not (the C-ABI
side of the boundary works on device pointers only), and it is what bench.py times as `e2e`.
"""

from __future__ import annotations

import torch

import unicaattention_b200 as unica

_STREAMS: dict = {}


def _streams(device: torch.device):
    if device not in _STREAMS:
        _STREAMS[device] = (torch.cuda.Stream(device), torch.cuda.Stream(device))
    return _STREAMS[device]


def group_sizes(heads: int, largest: int | None = None) -> list[int]:
    """Heads per group, in order.  The copies in run back to back, a head's worth taking a little less time than its
    kernels, and a group can start when its last head has arrived: so the groups grow by one head at a time (1, 2, 3, ..:
    each is there by the time the one before it is done), then stay at `largest` (default: an eighth of the heads), and
    the last one is small because its copy out has no kernels to hide behind.
    40 heads, largest 4: 1, 2, 3, 4, 4, 4, 4, 4, 4, 4, 4, 2."""
    largest = max(1, -(-heads // 8)) if largest is None else max(1, largest)
    back = [min(2, largest)] if heads >= 4 else []
    room = heads - sum(back)
    front, size = [], 1
    while size < largest and sum(front) + size <= room:
        front.append(size)
        size += 1
    left = room - sum(front)
    middle = [largest] * (left // largest) + ([left % largest] if left % largest else [])
    return front + middle + back


def attention_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor | None = None,
                   device: torch.device | int | None = None, heads_per_group: int | None = None, **settings) -> torch.Tensor:
    """softmax(q k^T / sqrt(d)) v for q [batch, heads, n_queries, 128], k, v [batch, heads, n_keys, 128] in HOST memory
    (pinned memory, and batch 1 or a layout whose head slices are contiguous, for the copies to overlap the kernels).
    `settings`: kernel / tile settings as for attention(), e.g. **PRESETS["per_channel"]; rope= stays a GPU tensor.
    Returns `out` (made in pinned memory when not given), valid once the current stream of `device` has been
    synchronised: nothing here waits for the GPU."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("attention_host takes host tensors; use attention() for tensors on the GPU")
    if q.dim() != 4 or k.shape != v.shape or k.shape[:2] != q.shape[:2]:
        raise ValueError(f"q [batch, heads, n_queries, 128] and k, v [batch, heads, n_keys, 128] expected, "
                         f"got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    device = torch.device("cuda", torch.cuda.current_device() if device is None else device) if not isinstance(device, torch.device) else device
    batch, heads = q.shape[:2]
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    elif out.shape != q.shape or out.dtype != q.dtype or out.is_cuda:
        raise ValueError("out must be a host tensor like q")
    if heads_per_group is None:
        # the largest group: about an eighth of the heads, picked so that its blocks fill their last wave of SMs well
        kernel = settings.get("kernel", unica.DEFAULT_KERNEL)
        candidates = range(max(1, -(-heads // 10)), max(1, -(-heads // 6)) + 1)
        largest = max(candidates, key=lambda g: (round(unica.wave_plan(batch * g, q.shape[2], kernel, device)["efficiency"], 2), g))
        sizes = group_sizes(heads, largest)
    else:
        sizes = [min(heads_per_group, heads - f) for f in range(0, heads, heads_per_group)]
    with torch.cuda.device(device):
        compute = torch.cuda.current_stream(device)
        copy_in, copy_out = _streams(device)
        qd, kd, vd = (torch.empty(x.shape, dtype=x.dtype, device=device) for x in (q, k, v))
        copy_in.wait_stream(compute)  # the staging memory may still be in use by work queued before this call
        copy_out.wait_stream(compute)
        first = 0
        for size in sizes:
            piece = slice(first, first + size)
            first += size
            with torch.cuda.stream(copy_in):
                for dst, src in ((qd, q), (kd, k), (vd, v)):
                    dst[:, piece].copy_(src[:, piece], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(copy_in)
            compute.wait_event(arrived)
            result = unica.attention(qd[:, piece], kd[:, piece], vd[:, piece], **settings)
            done = torch.cuda.Event()
            done.record(compute)
            copy_out.wait_event(done)
            with torch.cuda.stream(copy_out):
                out[:, piece].copy_(result, non_blocking=True)
            result.record_stream(copy_out)  # keep its memory until the copy has run
        compute.wait_stream(copy_out)  # a synchronise of the current stream now covers the copies back
    return out
