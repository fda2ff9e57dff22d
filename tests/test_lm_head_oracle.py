"""CPU checks of the oracle's LM-head restatement (row-wise int8 quantisation and the certified
top-1): the properties the reference's certificate rests on, and the tie rule."""
from __future__ import annotations

import numpy as np
import torch

SEED = 1234


def _matrix(rows: int, seed: int) -> torch.Tensor:
    generator = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, 2048, generator=generator) * 0.02).to(torch.bfloat16)


def _hidden(seed: int) -> torch.Tensor:
    generator = torch.Generator().manual_seed(seed)
    return torch.randn(2048, generator=generator).to(torch.bfloat16)


def test_quantisation_follows_the_reference_rules(oracle):
    weight = _matrix(96, SEED)
    weight[5] = 0                                               # all-zero row: scale falls back to 1e-12 / 127
    q, scales, residual = oracle.lm_head_quantize(weight)
    w = weight.float()
    maximum = w.abs().amax(dim=1).clamp_min(1.0e-12)
    inverse = np.float32(1.0) / np.float32(127.0)
    want_scale = (maximum.numpy() * inverse).astype(np.float32)
    assert np.array_equal(scales.numpy(), want_scale)           # multiplication by fl(1/127), not division
    want_q = torch.clamp(torch.round(w / scales[:, None]), -127, 127).to(torch.int8)
    assert torch.equal(q, want_q)                               # round-half-even, clamped
    assert int(q.abs().max()) == 127 and torch.equal(q[5], torch.zeros(2048, dtype=torch.int8))
    true_norm = (w.double() - q.double() * scales.double()[:, None]).norm(dim=1)
    assert bool((residual.double() >= true_norm).all())         # rounded outwards ...
    assert bool((residual.double() <= true_norm * (1 + 2.0e-6) + 1e-30).all())   # ... by a few ULPs only


def test_certificate_finds_the_exact_top1(oracle):
    rows = 3000
    weight = _matrix(rows, SEED + 1)
    q, scales, residual = oracle.lm_head_quantize(weight)
    for case in range(4):
        hidden = _hidden(SEED + 10 + case)
        got = oracle.lm_head_certify(weight, q, scales, residual, hidden)
        exact = oracle.gemv(weight, hidden).float()             # canonical dot, rounded to BF16
        best = float(exact.max())
        want_token = int((exact == best).nonzero()[0])
        assert got["status"] == 0 and got["overflow"] == 0
        assert got["top1_token"] == want_token and got["top1_logit"] == best
        # bounds hold for every row: the FP64 logit lies inside [approx - e, approx + e]
        true_logits = weight.double() @ hidden.double()
        approx = (q.double() * scales.double()[:, None]) @ hidden.double()
        error = residual.double() * got["hidden_l2"]
        assert bool(((true_logits - approx).abs() <= error).all())
        # candidates: exactly the rows whose upper bound reaches the largest lower bound; exact logits there
        candidates = got["candidates"].long()
        assert want_token in candidates.tolist() and 1 <= got["candidate_count"] <= 1024
        assert torch.equal(got["logits"][candidates], exact[candidates])


def test_equal_logits_resolve_to_the_lowest_token(oracle):
    weight = _matrix(512, SEED + 2)
    hidden = _hidden(SEED + 20)
    exact = oracle.gemv(weight, hidden).float()
    winner = int(exact.argmax())
    weight[40] = weight[winner]
    weight[300] = weight[winner]                                # three identical rows
    q, scales, residual = oracle.lm_head_quantize(weight)
    got = oracle.lm_head_certify(weight, q, scales, residual, hidden)
    assert got["top1_token"] == min(40, 300, winner)


def test_more_than_1024_candidates_is_reported(oracle):
    weight = _matrix(1, SEED + 3).repeat(1500, 1).contiguous()  # every row identical: all are candidates
    hidden = _hidden(SEED + 30)
    q, scales, residual = oracle.lm_head_quantize(weight)
    got = oracle.lm_head_certify(weight, q, scales, residual, hidden)
    assert got["status"] == -8 and got["overflow"] == 1 and got["candidate_count"] == 1500
