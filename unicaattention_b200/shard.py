"""Head-sharded dispatch over the GPUs of one box: the reference's sequential head-splitting for VRAM
(unica/__init__.py:208-245) turned into one process per GPU, each computing a contiguous slice of heads.

Every head is independent (its own statistics, scales and outliers, summed in a fixed order), so a rank runs the
single-GPU path on its slice and the result is bit for bit that of one whole call.  The only exchange is the gather of
the output heads: one NCCL all-gather over NVLink (`torch.distributed`; `gloo` on CPU for tests).
"""

from __future__ import annotations

import torch


def head_slice(heads: int, rank: int, world: int) -> slice:
    """Contiguous heads of `rank`: the first heads % world ranks hold one more (30 heads on 8 GPUs: 4,4,4,4,4,4,3,3)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(heads, world)
    first = rank * base + min(rank, extra)
    return slice(first, first + base + (1 if rank < extra else 0))


def gather_heads(local: torch.Tensor, out: torch.Tensor, heads: int, rank: int, world: int, group=None) -> torch.Tensor:
    """All-gather of each rank's [batch, its heads, tokens, 128] into out [batch, heads, tokens, 128] on every rank."""
    import torch.distributed as dist

    if out.shape[1] != heads or local.shape[1] != (s := head_slice(heads, rank, world)).stop - s.start:
        raise ValueError(f"rank {rank} holds {local.shape[1]} heads, expected {head_slice(heads, rank, world)} of {heads}")
    batch = out.shape[0]
    if heads % world == 0 and batch == 1 and out.is_contiguous() and local.is_contiguous():
        dist.all_gather_into_tensor(out.view(-1), local.view(-1), group=group)  # one collective, no staging copy
        return out
    # uneven slices or a batch dimension: equal-sized staging buffers (the smaller slices padded), then placement
    most = -(-heads // world)
    padded = local if local.shape[1] == most else torch.cat([local, local.new_zeros(batch, most - local.shape[1], *local.shape[2:])], 1)
    staged = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(staged, padded.contiguous(), group=group)
    for r, piece in enumerate(staged):
        s_ = head_slice(heads, r, world)
        out[:, s_].copy_(piece[:, : s_.stop - s_.start])
    return out


def slice_heads(inputs, heads: slice):
    """The operands kernel_inputs() returned, narrowed to a slice of their heads (every tensor in them is
    [batch, heads, ...]; tuples keep their type; numbers pass through)."""
    if isinstance(inputs, torch.Tensor):
        return inputs[:, heads] if inputs.dim() >= 2 else inputs
    if isinstance(inputs, tuple):
        parts = [slice_heads(x, heads) for x in inputs]
        return type(inputs)(*parts) if hasattr(inputs, "_fields") else tuple(parts)
    return inputs


_SIDE_STREAMS: dict = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    if device not in _SIDE_STREAMS:
        _SIDE_STREAMS[device] = torch.cuda.Stream(device, priority=-1)  # its few blocks go ahead of the attention kernel's
    return _SIDE_STREAMS[device]


def attention_sharded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, group=None, out: torch.Tensor | None = None,
                      head_groups: int | None = None, attention=None, kernel_inputs=None, **preset) -> torch.Tensor:
    """q, k, v: this rank's heads [batch, head_slice(heads, rank, world), tokens, 128].  Returns the whole
    [batch, heads, n_queries, 128] output on every rank (in `out` when given).

    The rank's heads are quantized once and then run through the attention kernel in `head_groups` groups (default: up to
    5); each group's output is gathered (one all-gather into a staging buffer, one strided copy into place) on a side
    stream while the next group's kernel runs, so that only the last group's gather is exposed.  Every head has its own
    statistics and scales, so the result is bit for bit that of one launch.  With a batch dimension, uneven head slices
    or head_groups = 1 the heads go through in one launch and one gather.
    attention / kernel_inputs: the functions to call (default: this package's; tests pass stand-ins)."""
    import torch.distributed as dist

    import unicaattention_b200 as unica

    attention = attention or unica.attention
    kernel_inputs = kernel_inputs or unica.kernel_inputs
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    batch, local_heads = q.shape[:2]
    if out is None:
        out = torch.empty((batch, heads, q.shape[2], q.shape[3]), dtype=q.dtype, device=q.device)
    groups = min(local_heads, 5) if head_groups is None else max(1, min(local_heads, head_groups))
    if groups == 1 or batch != 1 or heads % world or not q.is_cuda or not out.is_contiguous():
        return gather_heads(attention(q, k, v, **preset).contiguous(), out, heads, rank, world, group)
    inputs = kernel_inputs(q, k, v, **preset)
    current, side = torch.cuda.current_stream(q.device), _side_stream(q.device)
    side.wait_stream(current)  # `out` may still be read by work queued before this call
    placed = out.view(world, local_heads, *out.shape[2:])  # [rank, head of the rank, token, channel]
    base, extra = divmod(local_heads, groups)
    first = 0
    for g in range(groups):
        piece = slice(first, first + base + (1 if g < extra else 0))
        first = piece.stop
        local = attention(q[:, piece], k[:, piece], v[:, piece], inputs=slice_heads(inputs, piece), **preset)
        done = torch.cuda.Event()
        done.record(current)
        with torch.cuda.stream(side):
            side.wait_event(done)
            staged = torch.empty((world, piece.stop - piece.start, *out.shape[2:]), dtype=out.dtype, device=out.device)
            dist.all_gather_into_tensor(staged.view(-1), local.view(-1), group=group)
            placed[:, piece].copy_(staged)
        local.record_stream(side)
        staged.record_stream(current)
    current.wait_stream(side)
    return out
