"""CPU tests of the view scheduler's host logic: sharding arithmetic, and the broadcast +
shard protocol over a world_size-2 gloo group (no GPU, no kernels)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from renderformer_cuda_b200 import session


def test_shard_views_partitions_every_view_once():
    for n, world in [(64, 8), (64, 3), (5, 8), (0, 2), (7, 1)]:
        seen = []
        for r in range(world):
            mine = session.shard_views(n, r, world)
            assert all(v % world == r for v in mine)
            seen += mine
        assert sorted(seen) == list(range(n))
        sizes = [len(session.shard_views(n, r, world)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # the scene state travels as one byte blob from rank 0; every rank ends with identical bytes
    state = torch.arange(4096, dtype=torch.uint8) if rank == 0 else torch.zeros(4096, dtype=torch.uint8)
    dist.broadcast(state, src=0)
    mine = session.shard_views(11, rank, world)
    # a stand-in "render": each rank fills its own views, then the host gathers them
    frames = torch.zeros(11, 4)
    for v in mine:
        frames[v] = float(v) + state[:4].float()
    dist.all_reduce(frames)
    ret[rank] = (int(state.sum()), mine, frames.tolist())
    dist.destroy_process_group()


def test_broadcast_and_shard_protocol_gloo_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret[0][0] == ret[1][0] == int(torch.arange(4096, dtype=torch.uint8).sum())
    assert ret[0][1] == [0, 2, 4, 6, 8, 10] and ret[1][1] == [1, 3, 5, 7, 9]
    want = [[float(v) + i for i in range(4)] for v in range(11)]
    assert ret[0][2] == want and ret[1][2] == want
