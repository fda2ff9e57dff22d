"""CPU tests: the C oracle against the committed golden vectors (torch-CPU statement of the
reference's Python MoE path, tests/golden/make_golden.py) for BASELINE config 0."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"

# Stated tolerances (BASELINE north_star): max-abs <= 2e-2 and cosine >= 0.9999 on the layer's MoE
# output (routed + shared, before the residual add; after the add one BF16 ulp of an N(0,1)
# residual already exceeds 2e-2 for |x| >= 4, so the final hidden is held to MAX_ABS plus one ulp).
MAX_ABS = 2.0e-2
COSINE = 0.9999


def _load(tokens):
    data = np.load(GOLDEN / f"config0_T{tokens}.npz")
    seed, layer, count = (int(v) for v in data["seed"])
    assert count == tokens
    return data, seed, layer


def _bf16(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def _cosine(a, b):
    a, b = a.double().reshape(-1), b.double().reshape(-1)
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-30))


@pytest.mark.parametrize("tokens", [1, 16])
def test_prefill_oracle_matches_torch_golden(oracle, synth, tokens):
    data, seed, layer = _load(tokens)
    h2 = synth.activations(seed, tokens, "input", layer)
    after_attn = synth.activations(seed, tokens, "residual", layer)
    small = synth.layer_small_weights(seed, layer)

    routing = oracle.router_prefill(h2, oracle.OracleLayer({**small, "expert_gate_up_by_id": {},
                                                            "expert_down_by_id": {}}))
    # logits: same values up to BF16 rounding flips from FP32 summation order
    golden_logits = _bf16(data["logits"]).float()
    assert (routing["logits"] - golden_logits).abs().max() <= 2.0 ** -6
    assert (routing["logits"] == golden_logits).float().mean() > 0.97

    # the selection rule applied to torch's own logits must give torch.topk's values, and its set
    # wherever the 8th and 9th values differ
    forced = oracle.topk_prefill(golden_logits)
    assert torch.equal(forced["scores"], torch.from_numpy(data["topk_scores"]))
    sorted_logits = golden_logits.sort(dim=-1, descending=True).values
    untied = sorted_logits[:, 7] > sorted_logits[:, 8]
    golden_sets = torch.from_numpy(data["topk_indices"]).sort(dim=-1).values
    assert torch.equal(forced["ids"].long().sort(dim=-1).values[untied], golden_sets[untied])
    assert torch.equal(forced["weights"], _bf16(data["weights"]))

    experts = sorted(set(routing["ids"].reshape(-1).tolist()))
    weights = synth.layer_weights_cpu(seed, layer, experts)
    result = oracle.prefill_layer(h2, after_attn, oracle.OracleLayer(weights))
    assert torch.equal(result["ids"], routing["ids"])

    same_set = (result["ids"].long().sort(dim=-1).values == golden_sets).all(dim=-1)
    assert same_set.float().mean() >= 0.9
    golden_moe = (_bf16(data["moe_out"]).float() + _bf16(data["shared_out"]).float())
    oracle_moe = (result["routed"].float() + result["shared_scaled"].float())
    rows = same_set.nonzero().reshape(-1)
    assert (oracle_moe[rows] - golden_moe[rows]).abs().max() <= MAX_ABS
    assert _cosine(oracle_moe[rows], golden_moe[rows]) >= COSINE
    golden_out = _bf16(data["out"]).float()
    ulp = golden_out.abs().clamp_min(2.0 ** -126) * 2.0 ** -7
    assert ((result["out"].float() - golden_out).abs()[rows] <= ulp[rows] + MAX_ABS).all()


def test_decode_oracle_matches_torch_golden(oracle, synth):
    """The decode statement (FP32 logits, single final rounding) agrees with the torch path of the
    same layer within the stated tolerance; T = 1."""
    data, seed, layer = _load(1)
    h2_golden_input = synth.activations(seed, 1, "input", layer)      # what the torch path normalised
    after_attn = synth.activations(seed, 1, "residual", layer)
    small = synth.layer_small_weights(seed, layer)
    # decode forms h2 itself: feed a residual stream whose norm is the golden h2 is impossible in
    # general, so compare through a unit norm weight of zero and the golden h2 as residual stream
    small = dict(small)
    small["post_attention_layernorm"] = torch.zeros(2048, dtype=torch.bfloat16)
    probe = oracle.OracleLayer({**small, "expert_gate_up_by_id": {}, "expert_down_by_id": {}})
    ids = oracle.router_ids_decode(h2_golden_input[0], probe)
    weights = synth.layer_weights_cpu(seed, layer, ids.tolist())
    weights["post_attention_layernorm"] = small["post_attention_layernorm"]
    result = oracle.decode_layer(h2_golden_input[0], oracle.OracleLayer(weights))
    # same routed computation through the torch statement on the oracle's own h2
    import moe_torch_ref as ref

    h2 = result["h2"].reshape(1, 2048)
    compact = dict(small)
    order = result["ids"].tolist()
    compact["expert_gate_up"] = torch.stack([weights["expert_gate_up_by_id"][e] for e in order])
    compact["expert_down"] = torch.stack([weights["expert_down_by_id"][e] for e in order])
    moe = ref.expanded_routed_moe(h2, result["scores"].reshape(1, 8), torch.arange(8).reshape(1, 8), compact)
    shared = ref.shared_expert(h2, small)
    want = moe.float() + shared.float()
    got = result["routed"].float() + result["shared_scaled"].float()
    assert (got - want[0]).abs().max() <= MAX_ABS
    assert _cosine(got, want[0]) >= COSINE
    del after_attn
