"""GPU tests of the tensor-core (tcgen05) product kernel through the C ABI: the reference's
all-ones known answer, agreement with an FP32 torch reference, and agreement of the whole prefill
layer with the CUDA-core cross-check kernel at a size the CPU oracle cannot reach."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

SEED = 1234


@pytest.fixture(scope="module")
def provider(package, built_library):
    provider = package.MoeProvider(layers=1, max_prefill_tokens=0)
    yield provider
    provider.release()


def test_all_ones_gemm_reference_shape(provider):
    """native/src/bf16_gemm.hip.cpp:281-291: 8192 x 12352 x 2048 all-ones -> every output BF16 0x4500."""
    device = torch.device("cuda", 0)
    a = torch.ones(8192, 2048, dtype=torch.bfloat16, device=device)
    b = torch.ones(12352, 2048, dtype=torch.bfloat16, device=device)
    d = provider.gemm(a, b)
    provider.sync_metrics()
    bits = d.view(torch.int16)
    assert int((bits != 0x4500).sum()) == 0


@pytest.mark.parametrize("shape", [(128, 256, 64), (1, 8, 64), (300, 1000, 512), (1024, 2048, 2048), (77, 264, 192)])
def test_gemm_matches_fp32_reference(provider, shape):
    device = torch.device("cuda", 0)
    m, n, k = shape
    generator = torch.Generator(device=device).manual_seed(SEED + m + n + k)
    a = torch.randn(m, k, generator=generator, device=device, dtype=torch.float32).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=generator, device=device, dtype=torch.float32) * 0.05).to(torch.bfloat16)
    d = provider.gemm(a, b)
    provider.sync_metrics()
    want = (a.float() @ b.float().t())
    got = d.float()
    # one BF16 rounding of an FP32-accumulated sum: within 2^-8 relative plus accumulation noise
    tolerance = want.abs() * 2.0 ** -8 + 1e-3 * (k ** 0.5) * 0.05
    assert ((got - want).abs() <= tolerance).all()
    cosine = float((got.double().reshape(-1) @ want.double().reshape(-1)) /
                   (got.double().norm() * want.double().norm()))
    assert cosine >= 0.99999


def test_prefill_tensor_core_products_match_cuda_core_products(package, gpu_layers, synth):
    """Whole prefill layer at T = 1024 with skewed routing: tcgen05 products vs the CUDA-core
    cross-check kernel (same rounding points, different FP32 accumulation order)."""
    device = torch.device("cuda", 0)
    tokens = 1024
    weights = gpu_layers(0)["cuda"]
    h2 = synth.activations(SEED + 77, tokens, "input", 0).to(device)
    resid = synth.activations(SEED + 77, tokens, "residual", 0).to(device)
    bias = synth.zipf_router_bias(SEED).to(device)
    outputs = []
    for flags in (0, package.provider.FLAG_SIMT_PRODUCTS, package.provider.FLAG_MATERIALIZED_DISPATCH):
        provider = package.MoeProvider(layers=1, max_prefill_tokens=tokens, flags=flags)
        try:
            provider.bind_layer(0, weights)
            provider.set_router_hooks(bias, quantize_eighths=False)
            views, tensors = provider.make_debug(tokens, prefill=True)
            out = provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0, debug=views)
            provider.sync_metrics()
            outputs.append((out.clone(), {k: v.clone() for k, v in tensors.items()}))
        finally:
            provider.release()
    (out_tc, dbg_tc), (out_simt, dbg_simt), (out_copy, dbg_copy) = outputs
    # gathering rows inside the kernel (default) instead of reading a materialised copy changes no bit
    assert torch.equal(out_copy, out_tc)
    assert torch.equal(dbg_copy["routed"], dbg_tc["routed"])
    assert torch.equal(dbg_tc["topk_ids"], dbg_simt["topk_ids"])
    assert torch.equal(dbg_tc["sorted_rows"], dbg_simt["sorted_rows"])
    counts = dbg_tc["expert_counts"]
    assert int(counts.max()) > 128 and int((counts == 0).sum()) >= 0      # multi-tile and ragged experts
    moe_tc = dbg_tc["routed"].float() + dbg_tc["shared_scaled"].float()
    moe_simt = dbg_simt["routed"].float() + dbg_simt["shared_scaled"].float()
    assert (moe_tc - moe_simt).abs().max() <= 2.0e-2
    cosine = float((moe_tc.double().reshape(-1) @ moe_simt.double().reshape(-1)) /
                   (moe_tc.double().norm() * moe_simt.double().norm()))
    assert cosine >= 0.9999
    assert (dbg_tc["routed"] == dbg_simt["routed"]).float().mean() > 0.9
    assert torch.isfinite(out_tc.float()).all()


@pytest.mark.parametrize("tokens,regime", [(300, "zipf"), (1024, "uniform"), (2048, "zipf"), (8192, "hot")])
def test_two_sm_products_equal_one_sm_products(package, gpu_layers, synth, tokens, regime):
    """The expert products in the two-SM form (tcgen05.mma.cta_group::2, a pair of blocks per 256-row tile)
    against the one-SM form (128-row tiles): same operands in the same K order, so the same bits -- with
    experts of fewer than 128 rows (the second block of the pair idle), of 129 .. 256 rows and of many
    tiles, and the dispatch plan identical apart from the tile size."""
    device = torch.device("cuda", 0)
    weights = gpu_layers(0)["cuda"]
    h2 = synth.activations(SEED + 5 + tokens, tokens, "input", 0).to(device)
    resid = synth.activations(SEED + 5 + tokens, tokens, "residual", 0).to(device)
    bias = {"zipf": synth.zipf_router_bias(SEED), "hot": synth.hot_expert_bias(range(3, 256, 32)), "uniform": None}[regime]
    results = []
    for flags in (0, package.provider.FLAG_TWO_SM_PRODUCTS):
        provider = package.MoeProvider(layers=1, max_prefill_tokens=tokens, flags=flags)
        try:
            provider.bind_layer(0, weights)
            provider.set_router_hooks(None if bias is None else bias.to(device), quantize_eighths=False)
            views, tensors = provider.make_debug(tokens, prefill=True, with_logits=False)
            out = provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0, debug=views)
            provider.sync_metrics()
            results.append((out.clone(), {k: v.clone() for k, v in tensors.items()}))
        finally:
            provider.release()
    (out_one, dbg_one), (out_pair, dbg_pair) = results
    for name in ("topk_ids", "sorted_rows", "expert_counts", "expert_offsets"):
        assert torch.equal(dbg_pair[name], dbg_one[name]), name
    assert torch.equal(dbg_pair["routed"], dbg_one["routed"])
    assert torch.equal(dbg_pair["shared_scaled"], dbg_one["shared_scaled"])
    assert torch.equal(out_pair, out_one)
    assert torch.isfinite(out_pair.float()).all()


def test_certified_router_equals_exact_router_at_full_size(package, gpu_layers, synth):
    """T = 8192, three routing regimes: the tensor-core-filtered router and the all-256 canonical
    router must select identical experts in identical order (size the CPU oracle cannot reach)."""
    device = torch.device("cuda", 0)
    tokens = 8192
    weights = gpu_layers(0)["cuda"]
    provider = package.MoeProvider(layers=1, max_prefill_tokens=tokens)
    try:
        provider.bind_layer(0, weights)
        for regime in ("uniform", "ties", "zipf"):
            bias = synth.zipf_router_bias(SEED).to(device) if regime == "zipf" else None
            provider.set_router_hooks(bias, quantize_eighths=(regime == "ties"))
            generator = torch.Generator(device=device).manual_seed(SEED + len(regime))
            h2 = torch.randn(tokens, 2048, generator=generator, device=device).to(torch.bfloat16)
            resid = torch.randn(tokens, 2048, generator=generator, device=device).to(torch.bfloat16)
            results = []
            before = provider.sync_metrics()
            for with_logits in (False, True):
                views, tensors = provider.make_debug(tokens, prefill=True, with_logits=with_logits)
                out = provider.launch_selected_moe(post_attention=h2, residual_hidden=resid, model_layer=0,
                                                   debug=views)
                metrics = provider.sync_metrics()
                results.append((out.clone(), tensors))
            (out_cert, cert), (out_exact, exact) = results
            assert torch.equal(cert["topk_ids"], exact["topk_ids"]), regime
            assert torch.equal(cert["topk_scores"], exact["topk_scores"]), regime
            assert torch.equal(cert["topk_weights"], exact["topk_weights"]), regime
            assert torch.equal(out_cert, out_exact), regime
            per_token = (metrics.router_candidates - before.router_candidates) / tokens
            assert 8.0 <= per_token <= 48.0, (regime, per_token)
    finally:
        provider.release()
