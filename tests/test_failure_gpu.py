"""Failure detection without faulting a GPU: every wait in the kernels has a time budget; when a
peer's contribution never arrives the kernel raises a status word and returns, the host reads
AIMA_MOE_ERR_TIMEOUT, and the context stays usable.  Here the missing peer is a buffer that nothing
writes (rank 0 of a world of two runs alone on one GPU).  Also: the same inputs give the same bits on
every run."""
from __future__ import annotations

import hashlib
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

SEED = 1234
H = 2048


def _digest(tensor: torch.Tensor) -> str:
    return hashlib.sha256(tensor.detach().cpu().contiguous().view(torch.int16).numpy().tobytes()).hexdigest()


def test_a_silent_peer_ends_in_a_timeout_status_and_the_context_survives(package, gpu_layers, synth):
    device = torch.device("cuda", 0)
    weights = gpu_layers(0)["cuda"]
    x = synth.activations(SEED + 7, 1, "residual", 0)[0].to(device)
    provider = package.MoeProvider(layers=1, world=2, rank=0)
    try:
        slab = dict(weights)
        slab["expert_gate_up"] = weights["expert_gate_up"][:128].contiguous()
        slab["expert_down"] = weights["expert_down"][:128].contiguous()
        provider.bind_layer(0, slab)
        own = torch.zeros(2, 8, H, dtype=torch.int64, device=device)     # nothing ever writes the peer's share
        peer = torch.zeros(2, 8, H, dtype=torch.int64, device=device)
        provider.ep_connect(0, pointer=own.data_ptr())
        provider.ep_connect(1, pointer=peer.data_ptr())
        started = time.perf_counter()
        provider.decode_layer(x, 0)
        with pytest.raises(package.AimaMoeError) as error:
            provider.sync_metrics()
        elapsed = time.perf_counter() - started
        assert error.value.status == -5                                   # AIMA_MOE_ERR_TIMEOUT
        assert 1.0 < elapsed < 30.0                                       # the 2 s budget, not a hang
        assert provider.sync_metrics().device_status == 0                 # status cleared, exchange area reset
    finally:
        provider.release()
    # the device and the library are still good: a single-GPU handle gives the oracle's bits
    single = package.MoeProvider(layers=1)
    try:
        single.bind_layer(0, weights)
        first = single.decode_layer(x, 0)
        single.sync_metrics()
        second = single.decode_layer(x, 0)
        single.sync_metrics()
        assert torch.equal(first, second)
    finally:
        single.release()


def test_outputs_are_identical_across_runs(package, gpu_layers, synth):
    device = torch.device("cuda", 0)
    weights = gpu_layers(0)["cuda"]
    tokens = 257
    provider = package.MoeProvider(layers=1, max_prefill_tokens=tokens)
    try:
        provider.bind_layer(0, weights)
        provider.set_router_hooks(synth.hot_expert_bias(range(5, 256, 32)).to(device), False)   # most experts empty
        h2 = synth.activations(SEED + 8, tokens, "input", 0).to(device)
        resid = synth.activations(SEED + 8, tokens, "residual", 0).to(device)
        x = synth.activations(SEED + 9, 1, "residual", 0)[0].to(device)
        prefill, decode = set(), set()
        for _ in range(3):
            out = provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0)
            provider.sync_metrics()
            prefill.add(_digest(out))
            decode.add(_digest(provider.decode_layer(x, 0)))
            provider.sync_metrics()
        assert len(prefill) == 1 and len(decode) == 1
    finally:
        provider.release()
