"""The launches of the C ABI are asynchronous, allocation-free calls on the caller's stream, so a
host may record them into a CUDA graph once and replay it per token / per chunk (the reference
replays its decode schedule through an executor, native/src/native_decode_executor.hip.cpp).
Checked here: a captured decode stack and a captured prefill layer replay to the same bits as
the direct calls, for inputs that change between replays."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

SEED = 1234


def test_decode_stack_replays_from_a_cuda_graph(package, gpu_layers, synth):
    device = torch.device("cuda", 0)
    provider = package.MoeProvider(layers=3, max_prefill_tokens=0)
    try:
        for layer in range(3):
            provider.bind_layer(layer, gpu_layers(layer)["cuda"])
        inputs = [synth.activations(SEED + 700 + i, 1, "residual", 0)[0].to(device) for i in range(3)]
        direct = []
        for x in inputs:
            y = torch.empty_like(x)
            provider.decode_stack(x, y, 0, 3)
            provider.sync_metrics()
            direct.append(y.clone())

        x_static = inputs[0].clone()
        y_static = torch.empty_like(x_static)
        stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            provider.decode_stack(x_static, y_static, 0, 3)       # warm-up on the capture stream
            stream.synchronize()
            graph.capture_begin()
            provider.decode_stack(x_static, y_static, 0, 3)
            graph.capture_end()
        stream.synchronize()
        for x, want in zip(inputs, direct):
            x_static.copy_(x)
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(y_static, want)
        assert provider.sync_metrics().device_status == 0
    finally:
        provider.release()


def test_prefill_layer_replays_from_a_cuda_graph(package, gpu_layers, synth):
    device = torch.device("cuda", 0)
    tokens = 192
    provider = package.MoeProvider(layers=1, max_prefill_tokens=tokens)
    try:
        provider.bind_layer(0, gpu_layers(0)["cuda"])
        cases = [(synth.activations(SEED + 800 + i, tokens, "input", 0).to(device),
                  synth.activations(SEED + 800 + i, tokens, "residual", 0).to(device)) for i in range(2)]
        direct = []
        for h2, resid in cases:
            out = provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0)
            provider.sync_metrics()
            direct.append(out.clone())

        h2_static = cases[0][0].clone()
        resid_static = cases[0][1].clone()
        out_static = torch.empty_like(resid_static)
        stream = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            provider.launch_selected_moe(post_attention=h2_static, residual_hidden=resid_static,
                                         model_layer=0, out=out_static)
            stream.synchronize()
            graph.capture_begin()
            provider.launch_selected_moe(post_attention=h2_static, residual_hidden=resid_static,
                                         model_layer=0, out=out_static)
            graph.capture_end()
        stream.synchronize()
        for (h2, resid), want in zip(cases, direct):
            h2_static.copy_(h2)
            resid_static.copy_(resid)
            torch.cuda.synchronize()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out_static, want)
        assert provider.sync_metrics().device_status == 0
    finally:
        provider.release()
