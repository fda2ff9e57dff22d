"""One process driving two GPUs (skipped with fewer than two): every kernel's opt-in to more than
48 KB of dynamic shared memory is an attribute of the (function, device) pair, so the first launch
on the second device needs its own opt-in.  Each device runs on its own memory with plain loads
only -- no peer access -- through the handle API (decode and a prefill layer) and through the
allocation-free entry point; both devices must give the same bits.  A handle used while another
device is current is refused on the host."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

SEED = 2468


def _run_on(package, index: int):
    device = torch.device("cuda", index)
    with torch.cuda.device(device):
        weights = [package.synth.layer_weights_cuda_fast(SEED, layer, device) for layer in range(2)]
        provider = package.MoeProvider(layers=2, max_prefill_tokens=64)
        try:
            for layer, tensors in enumerate(weights):
                provider.bind_layer(layer, tensors)
            x = package.synth.activations(SEED, 1, "residual", 0)[0].to(device)
            decoded = torch.empty_like(x)
            provider.decode_stack(x, decoded, first_layer=0, n_layers=2)
            provider.sync_metrics()
            h2 = package.synth.activations(SEED, 33, "input", 0).to(device)
            resid = package.synth.activations(SEED, 33, "residual", 0).to(device)
            prefilled = provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0)
            provider.sync_metrics()
            status = torch.full((1,), -1, dtype=torch.int32, device=device)
            static = torch.zeros_like(x)
            package.provider.decode_layers_noalloc(weights, x, static, device_status=status)
            torch.cuda.synchronize(device)
            assert int(status.item()) == 0
            return decoded.cpu(), prefilled.cpu(), static.cpu(), provider
        except Exception:
            provider.release()
            raise


def test_one_process_drives_two_devices(package, built_library):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    first = _run_on(package, 0)
    second = _run_on(package, 1)
    try:
        assert torch.equal(first[0], second[0]), "decode differs between the devices"
        assert torch.equal(first[1], second[1]), "prefill differs between the devices"
        assert torch.equal(first[2], second[2]) and torch.equal(first[0], first[2])
        # a handle prepared on device 1 is refused while device 0 is current
        with torch.cuda.device(0):
            x = package.synth.activations(SEED, 1, "residual", 0)[0].to("cuda:0")
            with pytest.raises(package.AimaMoeError) as wrong_device:
                second[3].decode_layer(x, 0)
            assert wrong_device.value.status == -1
    finally:
        with torch.cuda.device(0):
            first[3].release()
        with torch.cuda.device(1):
            second[3].release()
