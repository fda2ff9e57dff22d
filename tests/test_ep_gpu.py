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


def test_expert_parallel_prefill_rank_alone_matches_single_gpu(package, gpu_layers, synth):
    """World of two on one GPU, one rank at a time: the peer's routing table, its staged
    activations, its flags and the rows it would return are written beforehand from a single-GPU
    run; the rank's output rows and the rows it returns must equal the single-GPU bits."""
    import ctypes

    device = torch.device("cuda", 0)
    weights = gpu_layers(0)["cuda"]
    total, per_rank = 192, 96
    h2 = synth.activations(SEED + 61, total, "input", 0).to(device)
    resid = synth.activations(SEED + 61, total, "residual", 0).to(device)

    single = package.MoeProvider(layers=1, max_prefill_tokens=total)
    try:
        single.bind_layer(0, weights)
        views, ref = single.make_debug(total, prefill=True, with_logits=False, with_slot_rows=True)
        want = single.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0, debug=views)
        single.sync_metrics()
        want = want.clone()
        ref = {k: v.clone() for k, v in ref.items()}
    finally:
        single.release()
    ids_all = ref["topk_ids"].reshape(-1)                       # [total * 8]
    weights_all = ref["topk_weights"].float().reshape(-1)

    for rank in (0, 1):
        lo, hi = rank * 128, rank * 128 + 128
        t0, t1 = rank * per_rank, (rank + 1) * per_rank
        other = 1 - rank
        o0, o1 = other * per_rank, (other + 1) * per_rank
        provider = package.MoeProvider(layers=1, max_prefill_tokens=total, world=2, rank=rank)
        try:
            slab = dict(weights)
            slab["expert_gate_up"] = weights["expert_gate_up"][lo:hi].contiguous()
            slab["expert_down"] = weights["expert_down"][lo:hi].contiguous()
            provider.bind_layer(0, slab)
            _, region_bytes = provider.ep_local_buffer()
            own = torch.zeros(region_bytes, dtype=torch.uint8, device=device)
            peer = torch.zeros(region_bytes, dtype=torch.uint8, device=device)
            # region layout (bytes after the 262144-byte decode part): flags 256 + 256,
            # ids [total*8] i32, weights [total*8] f32, h2 [total, 2048] bf16, return rows [total*8, 2048] bf16
            base = 262144
            rows = total * 8
            def span(n):
                nonlocal cursor
                at = cursor
                cursor += (n + 255) // 256 * 256
                return at
            cursor = base
            off_flag_routing, off_flag_returned = span(64), span(64)
            off_ids, off_w = span(rows * 4), span(rows * 4)
            off_h2, off_ret = span(total * H * 2), span(rows * H * 2)
            assert cursor == region_bytes
            def view(buf, off, count, dtype):
                return buf[off:off + count * torch.empty((), dtype=dtype).element_size()].view(dtype)
            # what the peer would have left in this rank's region before its flags went up
            view(own, off_flag_routing, 8, torch.int32)[other] = 1
            view(own, off_flag_returned, 8, torch.int32)[other] = 1
            view(own, off_ids, rows, torch.int32)[other * per_rank * 8:(other + 1) * per_rank * 8] = ids_all[o0 * 8:o1 * 8]
            view(own, off_w, rows, torch.float32)[other * per_rank * 8:(other + 1) * per_rank * 8] = weights_all[o0 * 8:o1 * 8]
            ret = view(own, off_ret, per_rank * 8 * H, torch.bfloat16).view(per_rank * 8, H)
            mine_ids = ids_all[t0 * 8:t1 * 8]
            remote = (mine_ids < lo) | (mine_ids >= hi)
            ret[remote] = ref["slot_rows"][t0 * 8:t1 * 8][remote]
            # the peer's activations, which its all-gather stores into block `other` of this rank's table
            view(own, off_h2, total * H, torch.bfloat16).view(total, H)[o0:o1].copy_(h2[o0:o1])
            provider.ep_connect(rank, pointer=own.data_ptr())
            provider.ep_connect(other, pointer=peer.data_ptr())
            out = provider.launch_selected_moe(post_attention=h2[t0:t1].contiguous(),
                                               residual_hidden=resid[t0:t1].contiguous(), model_layer=0)
            provider.sync_metrics()
            assert torch.equal(out, want[t0:t1]), f"rank {rank}"
            # rows this rank computed for the peer's tokens, as left in the peer's return area
            sent = view(peer, off_ret, per_rank * 8 * H, torch.bfloat16).view(per_rank * 8, H)
            peer_ids = ids_all[o0 * 8:o1 * 8]
            local = (peer_ids >= lo) & (peer_ids < hi)
            assert torch.equal(sent[local], ref["slot_rows"][o0 * 8:o1 * 8][local]), f"rank {rank} returned rows"
            # and this rank's own activations, stored into block `rank` of the peer's table
            assert torch.equal(view(peer, off_h2, total * H, torch.bfloat16).view(total, H)[t0:t1], h2[t0:t1])
            assert int(view(peer, off_flag_routing, 8, torch.int32)[rank]) == 1
            assert int(view(peer, off_flag_returned, 8, torch.int32)[rank]) == 1
        finally:
            provider.release()
    del ctypes


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _bits(tensor):
    """BF16 tensor as a numpy uint16 array: pickled by value, so the queue needs no shared file descriptors."""
    return tensor.detach().cpu().contiguous().view(torch.int16).numpy().copy()


def _from_bits(array):
    return torch.from_numpy(array).view(torch.bfloat16)


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
            outputs.append(_bits(y))
            x, y = y, x
        dist.barrier()
        # a soak of the hand-overs across GPUs: 600 more free-running steps with no host barrier between them
        # (ranks run ahead of one another as the tags allow); every rank must end with the same bits
        for _ in range(600):
            provider.decode_stack(x, y, 0, 3)
            x, y = y, x
        metrics = provider.sync_metrics()
        if metrics.device_status != 0:
            raise AssertionError(f"rank {rank}: device status {metrics.device_status} after the soak")
        soak = _bits(x)
        dist.barrier()
        provider.release()
        # prefill: 128 tokens per rank through layer 0
        prefill = package.MoeProvider(layers=1, max_prefill_tokens=128 * world, world=world, rank=rank)
        prefill.bind_layer(0, keep[0])
        prefill.ep_connect_all()
        h2_all = synth.activations(SEED + 77, 128 * world, "input", 0)
        resid_all = synth.activations(SEED + 77, 128 * world, "residual", 0)
        dist.barrier()
        out = prefill.launch_selected_moe(post_attention=h2_all[rank * 128:(rank + 1) * 128].to(device),
                                          residual_hidden=resid_all[rank * 128:(rank + 1) * 128].to(device),
                                          model_layer=0)
        prefill.sync_metrics()
        dist.barrier()
        outputs.append(_bits(out))
        prefill.release()
        # the pipelined variant (dispatch / products / return in two parts on three streams): same bits
        piped = package.MoeProvider(layers=1, max_prefill_tokens=128 * world, world=world, rank=rank,
                                    flags=package.provider.FLAG_EP_PIPELINE_2)
        piped.bind_layer(0, keep[0])
        piped.ep_connect_all()
        dist.barrier()
        again = piped.launch_selected_moe(post_attention=h2_all[rank * 128:(rank + 1) * 128].to(device),
                                          residual_hidden=resid_all[rank * 128:(rank + 1) * 128].to(device),
                                          model_layer=0)
        piped.sync_metrics()
        dist.barrier()
        if not torch.equal(again, out):
            raise AssertionError(f"rank {rank}: pipelined expert-parallel prefill differs from the plain one")
        piped.release()
        outputs.append(soak)
        results.put((rank, outputs))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_ranks_match_the_oracle(oracle, synth, world):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    context = mp.get_context("spawn")
    results = context.Queue()
    port = _free_port()
    processes = [context.Process(target=_rank_main, args=(rank, world, port, results)) for rank in range(world)]
    for process in processes:
        process.start()
    got = dict(results.get(timeout=600) for _ in range(world))
    got = {rank: [_from_bits(a) for a in arrays] for rank, arrays in got.items()}
    for process in processes:
        process.join(timeout=120)
        assert process.exitcode == 0
    layers = [oracle.OracleLayer(synth.layer_weights_cpu(SEED, layer)) for layer in range(3)]
    expected = synth.activations(SEED + 300, 1, "residual", 0)[0]
    for step in range(3):
        for layer in layers:
            expected = oracle.decode_layer(expected, layer)["out"]
        for rank in range(world):
            assert torch.equal(got[rank][step], expected), f"rank {rank} step {step}"
    for rank in range(1, world):
        assert torch.equal(got[rank][4], got[0][4]), f"rank {rank} differs from rank 0 after the soak"
    assert torch.isfinite(got[0][4].float()).all()
    # prefill rows of all ranks against the oracle (same tolerance as the single-GPU prefill tests)
    h2_all = synth.activations(SEED + 77, 128 * world, "input", 0)
    resid_all = synth.activations(SEED + 77, 128 * world, "residual", 0)
    select = sorted({0, 5, 127, 128, 200, 255, 128 * world - 1})
    want = oracle.prefill_layer(h2_all, resid_all, layers[0], select=select)
    everyone = torch.cat([got[rank][3] for rank in range(world)])
    ulp = want["out"].float().abs() * 2.0 ** -7
    assert ((everyone[select].float() - want["out"].float()).abs() <= ulp + 2.0e-2).all()
