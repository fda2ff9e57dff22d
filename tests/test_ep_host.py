"""CPU tests (gloo, world size 2) of the host side of expert parallelism: the bootstrap that carries
each rank's 64-byte IPC handle to every peer, and the expert slab arithmetic."""
from __future__ import annotations

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results) -> None:
    import conftest

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        package = conftest.load_package()
        mine = bytes((rank * 37 + i) % 256 for i in range(64))
        handles = package.provider.exchange_ipc_handles(mine, rank, world)
        results.put((rank, handles))
    finally:
        dist.destroy_process_group()


def test_ipc_handles_reach_every_rank_over_gloo():
    world = 2
    context = mp.get_context("spawn")
    results = context.Queue()
    port = _free_port()
    processes = [context.Process(target=_worker, args=(rank, world, port, results)) for rank in range(world)]
    for process in processes:
        process.start()
    got = dict(results.get(timeout=120) for _ in range(world))
    for process in processes:
        process.join(timeout=60)
        assert process.exitcode == 0
    expected = [bytes((rank * 37 + i) % 256 for i in range(64)) for rank in range(world)]
    assert got[0] == expected and got[1] == expected


def test_expert_slabs_partition_the_experts(synth):
    for world in (1, 2, 4, 8):
        per_rank = 256 // world
        owners = [e // per_rank for e in range(256)]
        assert sorted(set(owners)) == list(range(world))
        assert all(owners.count(r) == per_rank for r in range(world))
    # a rank's slab of the synthetic layer equals the same experts of the full layer
    full = synth.expert_down(1234, 0, 130)
    assert torch.equal(full, synth.expert_down(1234, 0, 130))
