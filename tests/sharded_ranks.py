"""One rank of a head-sharded job on real GPUs; started by test_gpu_multi.py (or by hand) as

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P tests/sharded_ranks.py

Every rank computes all heads by itself as the expected result, then its own slice through attention_sharded() with
both ways of gathering, and compares bit for bit.  Heads that do not divide by the ranks and a batch dimension are
included for the peer-store path, which supports them."""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import unicaattention_b200 as unica  # noqa: E402
from unicaattention_b200 import shard  # noqa: E402


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    checked = 0
    for batch, heads, n_queries in ((1, 2 * world, 1500), (1, 2 * world + 1, 700), (2, world, 300)):
        g = torch.Generator(device="cuda").manual_seed(11)  # the same tensors on every rank
        q, k, v = (torch.randn((batch, heads, n_queries, 128), device=device, dtype=torch.bfloat16, generator=g) for _ in range(3))
        mine = shard.head_slice(heads, rank, world)
        local_qkv = [x[:, mine].contiguous() for x in (q, k, v)]
        try:
            shared = shard.SharedOutput(batch, heads, n_queries)
        except RuntimeError as error:
            shared = None
            if rank == 0:
                print(f"no shared output: {error}", flush=True)
        for name, preset in unica.PRESETS.items():
            want = unica.attention(q, k, v, **preset)
            plain = shard.attention_sharded(*local_qkv, heads, **preset)
            assert torch.equal(plain, want), (name, "nccl", batch, heads)
            if shared is not None:
                shared.tensor.fill_(3.0)
                for _ in range(2):  # twice: the second call's stores meet the first call's result
                    got = shard.attention_sharded(*local_qkv, heads, out=shared, **preset)
                assert torch.equal(got, want), (name, "peer", batch, heads)
            checked += 1
        unica.check_status()
    dist.barrier()
    if rank == 0:
        print(f"sharded_ranks: {checked} cases equal on {world} ranks", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
