"""The certified prefill router under stress.  Its candidate filter rests on a bound on how far a
tensor-core FP32 logit can lie from the canonical one (kappa * |x| * |w|); the accumulation order of
the tensor cores is not published, so the bound is checked three ways:

* adversarial inputs -- rows scaled from 2^-8 to 2^8, alternating-sign rows of magnitude 256 whose
  products cancel, rows built to nearly cancel against one expert, router rows scaled by 50 -- over
  more than 64 K tokens: ids (order included), scores and weights equal those of the router that
  computes all 256 logits with the canonical dot;
* the kernel's own check of every candidate against the bound (router_bound_violations; a token that
  fails it is routed from all 256 canonical logits) -- reported;
* the audit flag: every 64th token routed both ways, mismatches counted -- must be zero.
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

SEED = 97531
T = 8192
FLAG_AUDIT_ROUTER = 256


@pytest.fixture(scope="module")
def provider(package, gpu_layers):
    weights = gpu_layers(0)["cuda"]
    scaled = dict(weights)
    scaled["router"] = (weights["router"].float() * 50.0).to(torch.bfloat16)
    provider = package.MoeProvider(layers=2, max_prefill_tokens=T, flags=FLAG_AUDIT_ROUTER)
    provider.bind_layer(0, weights)
    provider.bind_layer(1, scaled)
    provider._keep_scaled_router = scaled["router"]
    yield provider
    provider.release()


def _adversarial_rows(kind: str, router: torch.Tensor, seed: int) -> torch.Tensor:
    generator = torch.Generator().manual_seed(seed)
    base = torch.randn(T, 2048, generator=generator)
    if kind == "scaled":                       # N(0, 1) rows times 2^k, k = -8 .. 8
        exponent = torch.randint(-8, 9, (T, 1), generator=generator).float()
        rows = base * torch.pow(2.0, exponent)
    elif kind == "alternating":                # +-256 with a small perturbation: sum |x w| >> |sum x w|
        signs = torch.tensor([1.0, -1.0]).repeat(1024)
        rows = 256.0 * signs * (1.0 + 0.01 * base)
    elif kind == "cancelling":                 # large rows with the component along one expert's row removed
        w = router.float().cpu()
        target = torch.randint(0, 256, (T,), generator=generator)
        we = w[target]
        u = base * 64.0
        rows = u - ((u * we).sum(-1, keepdim=True) / (we * we).sum(-1, keepdim=True)) * we
    else:
        raise ValueError(kind)
    return rows.to(torch.bfloat16)


def _route(provider, layer, h2, exact: bool):
    device = torch.device("cuda", 0)
    views, tensors = provider.make_debug(T, prefill=True, with_logits=exact)     # the logits view selects the all-256 router
    provider.launch_selected_moe(post_attention=h2, residual_hidden=h2.clone(), model_layer=layer, debug=views)
    metrics = provider.sync_metrics()
    return {k: tensors[k].clone() for k in ("topk_ids", "topk_scores", "topk_weights")}, metrics


@pytest.mark.parametrize("layer", [0, 1], ids=["router", "router_x50"])
def test_certified_router_equals_the_exact_router_on_adversarial_rows(provider, gpu_layers, layer):
    device = torch.device("cuda", 0)
    router = gpu_layers(0)["cuda"]["router"]
    tokens = 0
    start = provider.sync_metrics()
    for kind in ("scaled", "alternating", "cancelling"):
        for repeat in range(2 if layer == 0 else 1):
            h2 = _adversarial_rows(kind, router, SEED + 10 * repeat + layer).to(device)
            certified, _ = _route(provider, layer, h2, exact=False)
            exact, _ = _route(provider, layer, h2, exact=True)
            for name in certified:
                assert torch.equal(certified[name], exact[name]), (kind, repeat, name)
            tokens += T
    end = provider.sync_metrics()
    audited = end.router_audited_tokens - start.router_audited_tokens
    assert audited >= tokens // 64
    assert end.router_audit_mismatches == start.router_audit_mismatches, "an audited token was routed differently"
    violations = end.router_bound_violations - start.router_bound_violations
    candidates = (end.router_candidates - start.router_candidates) / max(1, end.router_tokens - start.router_tokens)
    print(f"layer {layer}: {tokens} tokens, {candidates:.1f} candidates per token, {audited} audited, "
          f"{violations} tokens recomputed in full because a candidate broke the bound")
    assert tokens >= (49152 if layer == 0 else 24576)
