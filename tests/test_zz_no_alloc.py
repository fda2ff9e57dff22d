"""GPU test of the allocation-free decode entry point (collected last on purpose).

aima_moe_decode_layers_noalloc serves hosts that may not allocate device memory while they run
(all HBM already handed to their own arenas, or a request path on which cudaMalloc's device-wide
synchronisation is not acceptable).  It must give the same bits as the handle-based
aima_moe_decode_stack_launch and as the CPU oracle, on two calls in a row (the second call reuses
the static scratch array with the first call's contents in it), both in a fresh process and after
the other tests; it must leave the amount of free device memory unchanged; and it must turn away
memory that is not the current device's on the host, before anything is enqueued.
"""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "oracle"))
import moe_oracle  # noqa: E402  (the checker)

pytestmark = pytest.mark.gpu

SEED = 4321
LAYERS = 3


@pytest.fixture(scope="module")
def layers(package, built_library):
    device = torch.device("cuda", 0)
    return [package.synth.layer_weights_cuda_fast(SEED, layer, device) for layer in range(LAYERS)]


def test_noalloc_decode_matches_the_handle_based_entry_point(package, layers):
    device = torch.device("cuda", 0)
    provider = package.MoeProvider(layers=LAYERS)
    try:
        for layer, weights in enumerate(layers):
            provider.bind_layer(layer, weights)
        status = torch.full((1,), -1, dtype=torch.int32, device=device)
        views = [moe_oracle.OracleLayer({name: tensor.cpu() for name, tensor in weights.items()}) for weights in layers]
        for call in range(2):
            x = package.synth.activations(SEED + call, 1, "residual", 0)[0].to(device)
            want = torch.empty_like(x)
            provider.decode_stack(x, want, first_layer=0, n_layers=LAYERS)
            provider.sync_metrics()
            got = torch.zeros_like(x)
            package.provider.decode_layers_noalloc(layers, x, got, device_status=status)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            assert torch.equal(got, want), f"call {call}"          # bit-exact, as in the decode tests
            # and against the CPU oracle, layer by layer
            expected = x.cpu()
            for view in views:
                expected = moe_oracle.decode_layer(expected, view)["out"]
            assert torch.equal(got.cpu(), expected), f"call {call}: differs from the oracle"
            if call == 1:
                # the documented property itself: a call (after the first one on the device) leaves the
                # free device memory as it found it
                free_before, _ = torch.cuda.mem_get_info()
                package.provider.decode_layers_noalloc(layers, x, got, device_status=status)
                torch.cuda.synchronize()
                free_after, _ = torch.cuda.mem_get_info()
                assert free_after == free_before
        # a single layer through the static scratch as well
        x = package.synth.activations(SEED + 7, 1, "residual", 0)[0].to(device)
        want = provider.decode_layer(x, 1)
        got = torch.zeros_like(x)
        package.provider.decode_layers_noalloc([layers[1]], x, got)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    finally:
        provider.release()


def test_noalloc_decode_rejects_what_it_cannot_hold(package, layers):
    device = torch.device("cuda", 0)
    x = package.synth.activations(SEED, 1, "residual", 0)[0].to(device)
    y = torch.empty_like(x)
    too_many = [layers[0]] * (package.provider.NOALLOC_MAX_LAYERS + 1)
    with pytest.raises(package.AimaMoeError) as capacity:
        package.provider.decode_layers_noalloc(too_many, x, y)
    assert capacity.value.status == -8 and "AIMA_MOE_NOALLOC_MAX_LAYERS" in str(capacity.value)
    with pytest.raises(package.AimaMoeError) as alias:
        package.provider.decode_layers_noalloc([layers[0]], x, x)
    assert alias.value.status == -4
    without_norm = dict(layers[0])
    without_norm.pop("post_attention_layernorm")
    with pytest.raises(package.AimaMoeError) as missing:
        package.provider.decode_layers_noalloc([without_norm], x, y)
    assert missing.value.status == -1
    lib = package.load_library()
    assert lib.aima_moe_decode_layers_noalloc(None, 1, None, None, ctypes.c_float(1e-6), None, None) == -1
    # host memory for the vectors or for a weight: refused on the host with an error code, nothing enqueued
    # (raw pointers through the C ABI: the Python wrapper itself would refuse a CPU tensor)
    struct = package.provider.layer_weights_struct(layers[0])
    array = (type(struct) * 1)(struct)
    host_x = x.cpu()
    pointer = lambda tensor: ctypes.c_void_p(int(tensor.data_ptr()))
    status = lib.aima_moe_decode_layers_noalloc(array, 1, pointer(host_x), pointer(y), ctypes.c_float(1e-6), None, None)
    assert status == -1 and b"current device" in lib.aima_moe_last_error_string()
    host_router = layers[0]["router"].cpu()
    struct.router = pointer(host_router)
    array = (type(struct) * 1)(struct)
    status = lib.aima_moe_decode_layers_noalloc(array, 1, pointer(x), pointer(y), ctypes.c_float(1e-6), None, None)
    assert status == -1
    torch.cuda.synchronize()                                          # nothing ran, the context is untouched
    package.provider.decode_layers_noalloc([layers[0]], x, y)
    torch.cuda.synchronize()
