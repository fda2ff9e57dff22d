"""GPU parity of the batch-1 decode path through the C ABI: bit-exact against the CPU oracle
(routing ids, routing weights and every BF16 output), single layers and free-running stacks."""
from __future__ import annotations

import hashlib

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SEED = 1234


@pytest.fixture(scope="module")
def provider(package, gpu_layers):
    provider = package.MoeProvider(layers=4, max_prefill_tokens=0)
    for layer in range(3):
        provider.bind_layer(layer, gpu_layers(layer)["cuda"])
    yield provider
    provider.release()


def _decode_both(provider, oracle, gpu_layers, layer, x_cpu):
    device = torch.device("cuda", 0)
    views, tensors = provider.make_debug(1, prefill=False)
    out = provider.decode_layer(x_cpu.to(device), layer, debug=views)
    provider.sync_metrics()
    want = oracle.decode_layer(x_cpu, gpu_layers(layer)["oracle"])
    return out.cpu(), {k: v.cpu() for k, v in tensors.items()}, want


@pytest.mark.parametrize("case", range(6))
def test_decode_layer_is_bit_exact(provider, oracle, gpu_layers, synth, case):
    layer = case % 3
    x = synth.activations(SEED + case, 1, "residual", layer)[0]
    out, dbg, want = _decode_both(provider, oracle, gpu_layers, layer, x)
    assert torch.equal(dbg["h2"][0], want["h2"])
    assert torch.equal(dbg["router_logits"][0], want["logits"])       # FP32 bit patterns
    assert dbg["topk_ids"][0].tolist() == want["ids"].tolist()
    assert torch.equal(dbg["topk_scores"][0], want["scores"])
    assert torch.equal(dbg["topk_weights"][0], want["weights"])
    assert torch.equal(dbg["shared_scaled"][0], want["shared_scaled"])
    assert torch.equal(dbg["routed"][0], want["routed"])
    assert torch.equal(out, want["out"])


def test_decode_ties_resolve_to_the_lowest_expert(provider, oracle, gpu_layers, synth):
    """Logits rounded to multiples of 1/8 produce many exact ties (BASELINE config 4c)."""
    device = torch.device("cuda", 0)
    layer = 0
    provider.set_router_hooks(None, quantize_eighths=True)
    try:
        cpu = gpu_layers(layer)["cpu"]
        tied = oracle.OracleLayer(cpu, quant_eighths=True)
        ties_seen = 0
        for case in range(8):
            x = synth.activations(SEED + 100 + case, 1, "residual", layer)[0]
            views, tensors = provider.make_debug(1, prefill=False)
            out = provider.decode_layer(x.to(device), layer, debug=views)
            provider.sync_metrics()
            want = oracle.decode_layer(x, tied)
            assert tensors["topk_ids"][0].cpu().tolist() == want["ids"].tolist()
            assert torch.equal(out.cpu(), want["out"])
            scores = want["scores"].tolist()
            ties_seen += sum(1 for a, b in zip(scores, scores[1:]) if a == b)
        assert ties_seen > 0
    finally:
        provider.set_router_hooks(None, quantize_eighths=False)


def test_decode_router_bias_hook(provider, oracle, gpu_layers, synth):
    device = torch.device("cuda", 0)
    hot = [3, 40, 77, 101, 150, 199, 230, 255]
    bias = synth.hot_expert_bias(hot)
    provider.set_router_hooks(bias.to(device), quantize_eighths=False)
    try:
        x = synth.activations(SEED + 200, 1, "residual", 1)[0]
        views, tensors = provider.make_debug(1, prefill=False)
        out = provider.decode_layer(x.to(device), 1, debug=views)
        provider.sync_metrics()
        want = oracle.decode_layer(x, oracle.OracleLayer(gpu_layers(1)["cpu"], router_bias=bias))
        assert sorted(tensors["topk_ids"][0].cpu().tolist()) == hot
        assert tensors["topk_ids"][0].cpu().tolist() == want["ids"].tolist()
        assert torch.equal(out.cpu(), want["out"])
    finally:
        provider.set_router_hooks(None, quantize_eighths=False)


def test_decode_stack_free_running_is_bit_exact(provider, oracle, gpu_layers, synth):
    """Three layers chained inside one persistent launch, then fed back for several steps."""
    device = torch.device("cuda", 0)
    x = synth.activations(SEED + 300, 1, "residual", 0)[0]
    x_gpu = x.to(device)
    y_gpu = torch.empty_like(x_gpu)
    expected = x
    for step in range(4):
        provider.decode_stack(x_gpu, y_gpu, first_layer=0, n_layers=3)
        provider.sync_metrics()
        for layer in range(3):
            expected = oracle.decode_layer(expected, gpu_layers(layer)["oracle"])["out"]
        assert torch.equal(y_gpu.cpu(), expected), f"step {step}"
        x_gpu, y_gpu = y_gpu, x_gpu
    # the per-layer entry point gives the same result as the stack entry point
    z = x.to(device)
    for layer in range(3):
        z = provider.decode_layer(z, layer)
    single = oracle.decode_layer(x, gpu_layers(0)["oracle"])["out"]
    for layer in (1, 2):
        single = oracle.decode_layer(single, gpu_layers(layer)["oracle"])["out"]
    provider.sync_metrics()
    assert torch.equal(z.cpu(), single)


def test_words_between_layers_survive_the_wrap_of_their_tags(provider, gpu_layers, synth):
    """The words that carry a layer's output to the next layer hold a 16-bit tag, ((epoch) mod 65535) + 1.
    A stack launch at epoch E leaves words with the tags of E + 1 ..; a stack launch 65 535 epochs later expects
    exactly those tags again and must not take the old words for its own.  The epoch is preset with the
    qualification hook: the second launch gets a different input, and its result must be the one a launch
    at an unrelated epoch gives (single-layer launches in between, which advance the epoch without
    writing those words, are part of the scenario)."""
    device = torch.device("cuda", 0)
    x_a = synth.activations(SEED + 610, 1, "residual", 0)[0].to(device)
    x_b = synth.activations(SEED + 611, 1, "residual", 0)[0].to(device)
    out = torch.empty_like(x_a)
    provider.debug_set_decode_epoch(1000)
    provider.decode_stack(x_b, out, first_layer=0, n_layers=3)
    provider.sync_metrics()
    want_b = out.clone()
    provider.debug_set_decode_epoch(5000)
    provider.decode_stack(x_a, out, first_layer=0, n_layers=3)         # leaves words tagged for epochs 5001 ..
    provider.decode_layer(x_a, 0)                                       # a single-layer launch in between
    provider.sync_metrics()
    assert not torch.equal(out, want_b)
    for wraps in (1, 2):
        provider.debug_set_decode_epoch(5000 + wraps * 65535)           # the same tags come round
        provider.decode_stack(x_b, out, first_layer=0, n_layers=3)
        provider.sync_metrics()
        assert torch.equal(out, want_b), f"stale words of an earlier launch were read after {wraps} wrap(s)"
    provider.debug_set_decode_epoch(65535 * 65536 - 2)                  # the counter itself comes round inside a launch
    provider.decode_stack(x_b, out, first_layer=0, n_layers=3)
    provider.decode_stack(x_b, out, first_layer=0, n_layers=3)          # and the next launch starts from its small values
    provider.sync_metrics()
    assert torch.equal(out, want_b)


def test_decode_is_deterministic_across_runs(provider, gpu_layers, synth):
    device = torch.device("cuda", 0)
    x = synth.activations(SEED + 400, 1, "residual", 0)[0].to(device)
    digests = set()
    for _ in range(3):
        y = torch.empty_like(x)
        provider.decode_stack(x, y, first_layer=0, n_layers=3)
        provider.sync_metrics()
        digests.add(hashlib.sha256(y.cpu().view(torch.int16).numpy().tobytes()).hexdigest())
    assert len(digests) == 1


def test_two_thousand_free_running_steps_are_reproducible_with_and_without_prediction(package, gpu_layers, synth):
    """A soak of the hand-overs: 2000 tokens through a three-layer stack, each output fed back as the next input
    (18 000 grid-wide hand-overs by tagged words, the expert prediction right or wrong as the routing falls), run
    twice with prediction and once without: the three final vectors -- and the vectors after every 250th step --
    are the same bits, finite, and no bounded wait has run out.  A race between a writer and a late reader of
    an exchange word would show as a difference or as a timeout status."""
    device = torch.device("cuda", 0)
    runs = []
    for flags in (0, 0, package.provider.FLAG_NO_DECODE_PREDICTION):
        provider = package.MoeProvider(layers=3, max_prefill_tokens=0, flags=flags)
        try:
            for layer in range(3):
                provider.bind_layer(layer, gpu_layers(layer)["cuda"])
            buffers = [synth.activations(SEED + 900, 1, "residual", 0)[0].to(device), None]
            buffers[1] = torch.empty_like(buffers[0])
            checkpoints = []
            for step in range(2000):
                provider.decode_stack(buffers[step & 1], buffers[(step + 1) & 1], first_layer=0, n_layers=3)
                if step % 250 == 249:
                    # keep the residual stream bounded: the stack has no attention half to balance it
                    current = buffers[(step + 1) & 1]
                    checkpoints.append(current.clone())
                    current.copy_((current.float() / current.float().abs().max().clamp_min(1.0)).to(torch.bfloat16))
            metrics = provider.sync_metrics()
            assert metrics.device_status == 0
            runs.append(checkpoints)
        finally:
            provider.release()
    for a, b, c in zip(*runs):
        assert torch.isfinite(a.float()).all()
        assert torch.equal(a, b), "two runs with prediction differ"
        assert torch.equal(a, c), "prediction changed the result"


def test_decode_argument_checks(provider, package, synth):
    device = torch.device("cuda", 0)
    x = synth.activations(1, 1)[0].to(device)
    with pytest.raises(package.AimaMoeError) as alias:
        provider.decode_layer(x, 0, out=x)
    assert alias.value.status == -4
    with pytest.raises(package.AimaMoeError) as unbound:
        provider.decode_layer(x, 3)
    assert unbound.value.status == -3
    with pytest.raises(package.AimaMoeError):
        provider.decode_stack(x, torch.empty_like(x), first_layer=2, n_layers=5)


def _pattern(count, multiplier, increment, modulus, center, denominator):
    index = np.arange(count, dtype=np.uint64)
    integer = ((index * multiplier + increment) % modulus).astype(np.int64) - center
    return torch.from_numpy(integer.astype(np.float32) / np.float32(denominator)).to(torch.bfloat16)


@pytest.mark.parametrize("shape,digest", [
    ((2048, 512), "244856f006c62696b1dccd8c7882fc8d63e5063cdab825e8dcd8e4f0bf93cd0a"),
    ((2048, 4096), "7bfe6028c9df4e156947779c0aeb080ca8bfcc284def70e954e83bdb326db68b"),
])
def test_gemv_reproduces_reference_wvsplitk_hashes(provider, shape, digest):
    """Known-answer vectors of the reference's GEMV probe
    (native/src/bf16_wvsplitk.hip.cpp:218-333, benchmarks/results/native-wvsplitk-v0.1.0.json:52,73)."""
    device = torch.device("cuda", 0)
    m, k = shape
    weight = _pattern(m * k, 13, 7, 17, 8, 64.0).reshape(m, k).to(device)
    activation = _pattern(k, 11, 3, 19, 9, 32.0).to(device)
    out = provider.gemv(weight, activation)
    torch.cuda.synchronize()
    got = hashlib.sha256(out.cpu().view(torch.int16).numpy().tobytes()).hexdigest()
    assert got == digest


def test_rmsnorm_is_bit_exact(provider, oracle, synth):
    device = torch.device("cuda", 0)
    for rows in (1, 7, 33, 257):
        x = synth.activations(SEED + rows, rows)
        r = synth.activations(SEED + rows + 1, rows, "residual")
        w = synth.small_tensor("post_attention_layernorm", SEED, 0)
        _, n_gpu = provider.rmsnorm(x.to(device), w.to(device))
        _, n_cpu = oracle.rmsnorm(x, w)
        assert torch.equal(n_gpu.cpu(), n_cpu)
        r_gpu, n_gpu = provider.rmsnorm(x.to(device), w.to(device), residual=r.to(device))
        r_cpu, n_cpu = oracle.rmsnorm(x, w, residual=r)
        assert torch.equal(r_gpu.cpu(), r_cpu) and torch.equal(n_gpu.cpu(), n_cpu)
