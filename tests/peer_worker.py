"""One rank of the multi-GPU test of the peer-memory decode (launched by test_gpu_peer.py with
RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT set, NCCL backend, one GPU per rank).
Every rank encodes its shards into its symmetric-memory wire buffer, then decodes the whole
weight set - from the peers' buffers, from an NCCL all-gather, and through the overlapped
``WeightSetExchange`` step - and compares every result with the original tensors."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from losslessly_compressed_tensors_b200 import sharded  # noqa: E402
from losslessly_compressed_tensors_b200.comp_format import Distribution, DistType  # noqa: E402

SHAPES = [("emb", (2000, 96)), ("w1", (96, 384)), ("b1", (384,)), ("w2", (384, 96)), ("b2", (96,)),
          ("ln", (96,)), ("odd", (77, 1031))]


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=90),
                            device_id=torch.device("cuda", torch.cuda.current_device()))
    g = torch.Generator().manual_seed(5)
    tensors = []
    for i, (_, shape) in enumerate(SHAPES):
        w = torch.randn(shape, generator=g) * (30.0 if i == 6 else 0.02)
        if i == 6:
            w = w * torch.exp(torch.randn(shape, generator=g) * 4)   # overflow tails in the arena
        tensors.append(w.to(torch.bfloat16).cuda())
    plan = sharded.make_plan(SHAPES, world, Distribution(DistType.EMPIRICAL),
                             row_shard_elements=30000, arena_fraction=0.5)
    peer = sharded.PeerWire(plan, rank)
    shapes = [s for _, s in SHAPES]
    for step in range(3):                       # the same buffers are reused every step
        tensors[0].mul_(1.5)
        sharded.encode_rank(plan, rank, tensors, wire=peer.local)
        peer.fence()
        from_peers = sharded.decode_all(plan, peer.buffers, shapes, interleave_from=rank + 1)
        staged = sharded.decode_all(plan, peer.buffers, shapes, interleave_from=rank + 1,
                                    stage_remote_for=rank)   # side bytes through local scratch
        gathered = sharded.all_gather_wire(peer.local.clone(), plan)
        from_gather = sharded.decode_all(plan, gathered, shapes)
        peer.fence()
        for want, a, b, c in zip(tensors, from_peers, from_gather, staged):
            assert torch.equal(a.view(torch.int16), want.view(torch.int16)), (rank, step)
            assert torch.equal(c.view(torch.int16), want.view(torch.int16)), (rank, step)
            assert torch.equal(b.view(torch.int16), want.view(torch.int16)), (rank, step)
    # The overlapped step: one fence, source-by-source copies on a side stream, decode as they land.
    exchange = sharded.WeightSetExchange(plan, rank, tensors, shapes)
    for step in range(4):                       # both wire buffers are used twice
        tensors[1].add_(0.25)
        restored = exchange.step()
        torch.cuda.synchronize()
        for want, got in zip(tensors, restored):
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (rank, "exchange", step)
    torch.cuda.synchronize()
    dist.barrier()
    print(f"PEER-OK rank {rank} multicast_bound={peer.multicast}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
