"""GPU tests of expert-parallel decode.

One GPU: each rank of a world of two runs alone, with the other rank's contributions (per-slot down
products taken from a single-GPU run) written into its exchange buffer beforehand, exactly as the
peer's stores would leave them; the result must equal the single-GPU result bit for bit and the
values it sends must be the ones the peer needs.  (Two waiting kernels are never run at the same
time on one GPU.)  Two or more GPUs: real ranks as processes, handles carried over gloo."""
from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

SEED = 1234
H = 2048


def _tagged(values: torch.Tensor, tag: int) -> torch.Tensor:
    bits = values.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return bits | (tag << 32)


def test_expert_parallel_rank_alone_matches_single_gpu(package, gpu_layers, synth):
    device = torch.device("cuda", 0)
    layers = [gpu_layers(0)["cuda"], gpu_layers(1)["cuda"]]
    x = synth.activations(SEED + 5, 1, "residual", 0)[0].to(device)

    single = package.MoeProvider(layers=2)
    per_layer = []
    try:
        for layer, weights in enumerate(layers):
            single.bind_layer(layer, weights)
        current = x
        for layer in range(2):
            views, tensors = single.make_debug(1, prefill=False)
            current = single.decode_layer(current, layer, debug=views)
            single.sync_metrics()
            per_layer.append({"ids": tensors["topk_ids"][0].clone(), "dots": tensors["slot_dots"].clone()})
        want = torch.empty_like(x)
        single.decode_stack(x, want, 0, 2)
        single.sync_metrics()
        assert torch.equal(want, current)
    finally:
        single.release()

    for rank in (0, 1):
        lo, hi = rank * 128, rank * 128 + 128
        provider = package.MoeProvider(layers=2, world=2, rank=rank)
        try:
            for layer, weights in enumerate(layers):
                slab = dict(weights)
                slab["expert_gate_up"] = weights["expert_gate_up"][lo:hi].contiguous()
                slab["expert_down"] = weights["expert_down"][lo:hi].contiguous()
                provider.bind_layer(layer, slab)
            own = torch.zeros(2, 8, H, dtype=torch.int64, device=device)       # [parity][slot][h]
            peer = torch.zeros(2, 8, H, dtype=torch.int64, device=device)
            for layer in range(2):
                ids = per_layer[layer]["ids"].tolist()
                for slot, expert in enumerate(ids):
                    if not lo <= expert < hi:
                        own[layer & 1, slot] = _tagged(per_layer[layer]["dots"][slot], layer + 1)
            provider.ep_connect(rank, pointer=own.data_ptr())
            provider.ep_connect(1 - rank, pointer=peer.data_ptr())
            got = torch.empty_like(x)
            provider.decode_stack(x, got, 0, 2)
            provider.sync_metrics()
            assert torch.equal(got, want), f"rank {rank}"
            for layer in range(2):
                ids = per_layer[layer]["ids"].tolist()
                for slot, expert in enumerate(ids):
                    sent = peer[layer & 1, slot]
                    if lo <= expert < hi:
                        assert torch.equal(sent, _tagged(per_layer[layer]["dots"][slot], layer + 1)), (rank, layer, slot)
                    else:
                        assert int(sent.abs().sum()) == 0
        finally:
            provider.release()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, results) -> None:
    import torch.distributed as dist
    import conftest

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        package = conftest.load_package()
        synth = package.synth
        device = torch.device("cuda", rank)
        per_rank = 256 // world
        lo, hi = rank * per_rank, (rank + 1) * per_rank
        provider = package.MoeProvider(layers=3, world=world, rank=rank)
        keep = []
        for layer in range(3):
            weights = synth.layer_weights_cuda(SEED, layer, device, lo, hi)
            provider.bind_layer(layer, weights)
            keep.append(weights)
        provider.ep_connect_all()
        x = synth.activations(SEED + 300, 1, "residual", 0)[0].to(device)
        y = torch.empty_like(x)
        outputs = []
        for _ in range(3):
            dist.barrier()
            provider.decode_stack(x, y, 0, 3)
            provider.sync_metrics()
            outputs.append(y.cpu().clone())
            x, y = y, x
        dist.barrier()
        provider.release()
        results.put((rank, outputs))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_two_gpus_match_the_oracle(oracle, synth):
    import torch.multiprocessing as mp

    world = 2
    context = mp.get_context("spawn")
    results = context.Queue()
    port = _free_port()
    processes = [context.Process(target=_rank_main, args=(rank, world, port, results)) for rank in range(world)]
    for process in processes:
        process.start()
    got = dict(results.get(timeout=600) for _ in range(world))
    for process in processes:
        process.join(timeout=120)
        assert process.exitcode == 0
    layers = [oracle.OracleLayer(synth.layer_weights_cpu(SEED, layer)) for layer in range(3)]
    expected = synth.activations(SEED + 300, 1, "residual", 0)[0]
    for step in range(3):
        for layer in layers:
            expected = oracle.decode_layer(expected, layer)["out"]
        assert torch.equal(got[0][step], expected), f"rank 0 step {step}"
        assert torch.equal(got[1][step], expected), f"rank 1 step {step}"
