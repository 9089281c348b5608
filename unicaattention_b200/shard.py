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


def attention_sharded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, group=None, out: torch.Tensor | None = None,
                      **preset) -> torch.Tensor:
    """q, k, v: this rank's heads [batch, head_slice(heads, rank, world), tokens, 128].  Returns the whole
    [batch, heads, n_queries, 128] output on every rank (in `out` when given)."""
    import torch.distributed as dist

    import unicaattention_b200 as unica

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    local = unica.attention(q, k, v, **preset)
    if out is None:
        out = torch.empty((q.shape[0], heads, q.shape[2], q.shape[3]), dtype=q.dtype, device=q.device)
    return gather_heads(local.contiguous(), out, heads, rank, world, group)
