"""Head-sharded dispatch over the GPUs of one box: the reference's sequential head-splitting for VRAM
(unica/__init__.py:208-245) turned into one process per GPU, each computing a contiguous slice of heads.

Every head is independent (its own statistics, scales and outliers, summed in a fixed order), so a rank runs the
single-GPU path on its slice and the result is bit for bit that of one whole call.  The only exchange is the gather of
the output heads, done one of two ways:

- fused into the attention kernel: the output lives in memory every rank has mapped (SharedOutput) and each kernel
  stores the rows it computes into every rank's copy over NVLink as it finishes them, so no gather remains afterwards,
  only a barrier;
- NCCL all-gathers of groups of heads on a side stream while the next group computes (any output tensor; `gloo` on
  CPU for tests), which leaves the last group's gather exposed.
"""

from __future__ import annotations

import os

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


class SharedOutput:
    """An output tensor [batch, heads, tokens, 128] (bfloat16) in memory that every rank of `group` has mapped, made with
    torch's symmetric memory (a collective: every rank constructs it, with the same shape).  `tensor` is this rank's copy;
    `addresses[r]` is where rank r's copy starts in this process's address space.  The attention kernels only ever store
    to the other ranks' copies, with plain stores; the NVLink multicast binding torch would otherwise add is not
    needed and is switched off unless TORCH_SYMM_MEM_DISABLE_MULTICAST is already set.
    Raises RuntimeError where the ranks cannot map each other's memory (then use a plain tensor: the gather goes
    through NCCL)."""

    def __init__(self, batch: int, heads: int, tokens: int, group=None, device: torch.device | None = None) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world - 1 > 7:
            raise RuntimeError(f"the kernels store to at most 7 peers, the group has {self.world} ranks")
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.token = torch.zeros(1, dtype=torch.int32, device=device)  # what the barriers reduce
        try:
            self.tensor, error = symmetric.empty((batch, heads, tokens, 128), dtype=torch.bfloat16, device=device), None
        except Exception as e:  # torch raises several types here, depending on what the driver refused
            self.tensor, error = None, e
        refused = torch.tensor([error is not None], dtype=torch.int32, device=device)
        dist.all_reduce(refused, group=self.group)  # the ranks go on to the rendezvous together or not at all
        if int(refused):
            raise RuntimeError(f"no shared output on this machine: {error or 'another rank could not allocate it'}")
        try:
            self.handle = symmetric.rendezvous(self.tensor, self.group)
        except Exception as e:
            raise RuntimeError(f"no shared output on this machine: {e}") from e
        self.addresses = [int(a) for a in self.handle.buffer_ptrs]
        if len(self.addresses) != self.world or self.addresses[self.rank] != self.tensor.data_ptr():
            raise RuntimeError("symmetric memory returned addresses that do not match the group")

    def peers_of(self, view: torch.Tensor) -> list[int]:
        """Addresses of `view` (a view of self.tensor) in the other ranks' copies."""
        ahead = view.data_ptr() - self.tensor.data_ptr()
        return [a + ahead for r, a in enumerate(self.addresses) if r != self.rank]

    def barrier(self) -> None:
        """Every rank's work queued before this (on its current stream) is complete before any rank's work queued after
        it starts: one tiny all-reduce."""
        import torch.distributed as dist

        dist.all_reduce(self.token, group=self.group)


_SIDE_STREAMS: dict = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    if device not in _SIDE_STREAMS:
        _SIDE_STREAMS[device] = torch.cuda.Stream(device, priority=-1)  # its few blocks go ahead of the attention kernel's
    return _SIDE_STREAMS[device]


def attention_shared(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: SharedOutput, attention=None, kernel_inputs=None,
                     **preset) -> torch.Tensor:
    """attention_sharded() into a SharedOutput: one launch whose kernel stores this rank's heads into every rank's copy.
    Between two barriers: the first (on a side stream, hidden behind the quantization) keeps this call's stores from
    reaching a rank that still reads the previous result, the second ends when every rank's stores have landed.
    Uneven head slices and a batch dimension are fine: every row has one writer.  Returns out.tensor."""
    import unicaattention_b200 as unica

    attention = attention or unica.attention
    kernel_inputs = kernel_inputs or unica.kernel_inputs
    if q.dtype != torch.bfloat16:
        raise TypeError("a shared output takes bfloat16 q, k, v")
    heads = out.tensor.shape[1]
    mine = head_slice(heads, out.rank, out.world)
    if q.shape[1] != mine.stop - mine.start or q.shape[0] != out.tensor.shape[0] or q.shape[2] != out.tensor.shape[2]:
        raise ValueError(f"rank {out.rank} holds q {tuple(q.shape)}, expected heads {mine} of an output {tuple(out.tensor.shape)}")
    current, side = torch.cuda.current_stream(q.device), _side_stream(q.device)
    side.wait_stream(current)
    with torch.cuda.stream(side):
        out.barrier()
    inputs = kernel_inputs(q, k, v, **preset)
    current.wait_stream(side)
    view = out.tensor[:, mine]
    attention(q, k, v, inputs=inputs, out=view, peer_out=out.peers_of(view), **preset)
    out.barrier()
    return out.tensor


def attention_sharded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, group=None,
                      out: torch.Tensor | SharedOutput | None = None, head_groups: int | None = None, attention=None,
                      kernel_inputs=None, **preset) -> torch.Tensor:
    """q, k, v: this rank's heads [batch, head_slice(heads, rank, world), tokens, 128].  Returns the whole
    [batch, heads, n_queries, 128] output on every rank (in `out` when given).

    With a SharedOutput the gather is part of the kernel (attention_shared).  Otherwise the rank's heads are quantized once and then run through the attention kernel in `head_groups` groups (default: up to
    5); each group's output is gathered (one all-gather into a staging buffer, one strided copy into place) on a side
    stream while the next group's kernel runs, so that only the last group's gather is exposed.  Every head has its own
    statistics and scales, so the result is bit for bit that of one launch.  With a batch dimension, uneven head slices
    or head_groups = 1 the heads go through in one launch and one gather.
    attention / kernel_inputs: the functions to call (default: this package's; tests pass stand-ins)."""
    import torch.distributed as dist

    import unicaattention_b200 as unica

    if isinstance(out, SharedOutput):
        return attention_shared(q, k, v, out, attention, kernel_inputs, **preset)
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
