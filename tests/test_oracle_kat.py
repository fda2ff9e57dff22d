"""CPU tests that pin the oracle: the reference's own known-answer vectors, the
selection rules, and agreement with torch CPU operators."""
from __future__ import annotations

import hashlib
import math

import numpy as np
import pytest
import torch


def _pattern(count, multiplier, increment, modulus, center, denominator):
    # fill_pattern_kernel / pattern_value, native/src/bf16_wvsplitk.hip.cpp:218-247
    index = np.arange(count, dtype=np.uint64)
    integer = ((index * multiplier + increment) % modulus).astype(np.int64) - center
    return torch.from_numpy(integer.astype(np.float32) / np.float32(denominator)).to(torch.bfloat16)


# benchmarks/results/native-wvsplitk-v0.1.0.json:52,73 (output_bf16_sha256)
WVSPLITK_GOLDEN = {
    (2048, 512): "244856f006c62696b1dccd8c7882fc8d63e5063cdab825e8dcd8e4f0bf93cd0a",
    (2048, 4096): "7bfe6028c9df4e156947779c0aeb080ca8bfcc284def70e954e83bdb326db68b",
}


@pytest.mark.parametrize("shape", sorted(WVSPLITK_GOLDEN))
def test_gemv_reproduces_reference_wvsplitk_hashes(oracle, shape):
    m, k = shape
    weight = _pattern(m * k, 13, 7, 17, 8, 64.0).reshape(m, k)
    activation = _pattern(k, 11, 3, 19, 9, 32.0)
    out = oracle.gemv(weight, activation)
    digest = hashlib.sha256(oracle.bf16_numpy(out).tobytes()).hexdigest()
    assert digest == WVSPLITK_GOLDEN[shape]


def test_all_ones_dot_is_2048(oracle):
    # native/src/bf16_gemm.hip.cpp:281-291: all-ones operands with K = 2048 give BF16 0x4500
    ones = torch.ones(2048, dtype=torch.bfloat16)
    out = oracle.gemv(ones.reshape(1, 2048).repeat(4, 1), ones)
    assert oracle.bf16_numpy(out).tolist() == [0x4500] * 4


def test_deterministic_exp_accuracy(oracle):
    lib = oracle.lib()
    worst = 0.0
    for x in np.linspace(-30.0, 30.0, 6001, dtype=np.float32):
        got = lib.aima_or_expf(float(x))
        want = math.exp(float(x))
        worst = max(worst, abs(got - want) / want)
    assert worst < 4.0e-7          # within ~3 ulp of FP32
    assert lib.aima_or_expf(0.0) == 1.0


def test_rmsnorm_matches_torch(oracle, torch_ref, synth):
    x = synth.activations(7, 33)
    w = synth.small_tensor("post_attention_layernorm", 7, 0)
    _, got = oracle.rmsnorm(x, w)
    want = torch_ref.rmsnorm(x, w)
    diff = (got.float() - want.float()).abs()
    # identical up to BF16 rounding flips caused by a different FP32 summation order
    assert (diff <= want.float().abs() * 2.0 ** -7 + 1e-30).all()
    assert (got == want).float().mean() > 0.98
    resid = synth.activations(8, 33)
    r_out, n_out = oracle.rmsnorm(x, w, residual=resid)
    assert torch.equal(r_out, (x.float() + resid.float()).to(torch.bfloat16))
    _, n_ref = oracle.rmsnorm(r_out, w)
    assert torch.equal(n_out, n_ref)


def _reference_prefill_rule(row):
    """Independent numpy statement of router_topk8_softmax_256_kernel's ordering."""
    order = sorted(range(256), key=lambda e: (-row[e], e))
    threshold = row[order[7]]
    chosen = [e for e in range(256) if row[e] > threshold]
    chosen += [e for e in range(256) if row[e] == threshold][: 8 - len(chosen)]
    values = [row[e] for e in chosen]
    width = 2
    while width <= 8:
        stride = width // 2
        while stride > 0:
            for left in range(8):
                right = left ^ stride
                if right <= left:
                    continue
                ascending = (left & width) != 0
                if (values[left] > values[right]) == ascending:
                    values[left], values[right] = values[right], values[left]
                    chosen[left], chosen[right] = chosen[right], chosen[left]
            stride //= 2
        width *= 2
    return chosen, values


def test_selection_rules_on_ties(oracle):
    generator = torch.Generator().manual_seed(5)
    logits = torch.randn(400, 256, generator=generator)
    logits = (logits * 8).round() / 8            # many exact ties
    prefill = oracle.topk_prefill(logits)
    decode = oracle.topk_decode(logits)
    for t in range(logits.shape[0]):
        row = logits[t].tolist()
        chosen, values = _reference_prefill_rule(row)
        assert prefill["ids"][t].tolist() == chosen
        assert prefill["scores"][t].tolist() == values
        # decode rule: descending value, ties to the lowest id
        want = sorted(range(256), key=lambda e: (-row[e], e))[:8]
        assert decode["ids"][t].tolist() == want
        # both rules pick the same SET
        assert sorted(chosen) == sorted(want)
        assert values == sorted(values, reverse=True)
    # softmax weights: BF16 of exp(s - s0) / sum
    scores = prefill["scores"]
    want_w = torch.softmax(scores, dim=-1)
    assert (prefill["weights"].float() - want_w).abs().max() < 2.0 ** -8


def test_selection_without_ties_matches_torch_topk(oracle):
    generator = torch.Generator().manual_seed(6)
    logits = torch.randn(200, 256, generator=generator)
    values, indices = torch.topk(logits, 8, dim=-1)
    assert torch.equal(oracle.topk_decode(logits)["ids"].long(), indices)
    assert torch.equal(oracle.topk_prefill(logits)["ids"].long(), indices)
    assert torch.equal(oracle.topk_prefill(logits)["scores"], values)


def test_dispatch_plan_is_a_stable_sort(oracle, torch_ref):
    generator = torch.Generator().manual_seed(9)
    for tokens in (1, 7, 33, 257):
        ids = torch.stack([torch.randperm(256, generator=generator)[:8] for _ in range(tokens)]).int()
        plan = oracle.dispatch_plan(ids)
        table = torch_ref.build_dispatch_table(ids.long())
        assert torch.equal(plan["sorted_rows"].long(), table["active_positions"])
        assert int(plan["offsets"][-1]) == tokens * 8
        counts = torch.bincount(ids.reshape(-1).long(), minlength=256)
        assert torch.equal(plan["counts"].long(), counts)
        assert plan["padded_rows"] == int(((counts + 31) // 32 * 32).sum())
    # hot-expert case: every token picks the same eight experts
    ids = torch.arange(8, dtype=torch.int32).repeat(100, 1)
    plan = oracle.dispatch_plan(ids)
    assert plan["counts"][:8].tolist() == [100] * 8 and int(plan["counts"][8:].sum()) == 0
