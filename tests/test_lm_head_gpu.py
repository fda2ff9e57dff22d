"""GPU parity of the LM head with a certified top-1 through the C ABI: int8 copy, scales and
residual norms bit-exact against the CPU oracle, approximate logits bit-exact, the same candidate
set, the same exact top-1; at the reference's vocabulary size the certified token equals the
arg-max of the full exact BF16 GEMV."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

SEED = 1234


def _matrix(rows: int, seed: int) -> torch.Tensor:
    generator = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, 2048, generator=generator) * 0.02).to(torch.bfloat16)


def _hidden(seed: int) -> torch.Tensor:
    generator = torch.Generator().manual_seed(seed)
    return torch.randn(2048, generator=generator).to(torch.bfloat16)


def test_lm_head_matches_the_oracle(package, oracle):
    device = torch.device("cuda", 0)
    rows = 5000
    weight = _matrix(rows, SEED + 1)
    weight[7] = 0
    weight[4100] = weight[12]                                   # duplicate rows: ties
    q_want, scales_want, residual_want = oracle.lm_head_quantize(weight)
    head = package.LmHead(weight.to(device))
    try:
        q, scales, residual = head.views()
        assert torch.equal(q, q_want)
        assert torch.equal(scales, scales_want)
        assert torch.equal(residual, residual_want)
        for case in range(4):
            hidden = _hidden(SEED + 50 + case)
            want = oracle.lm_head_certify(weight, q_want, scales_want, residual_want, hidden)
            logits = head.launch(hidden.to(device))
            result = head.result()
            assert result.hidden_l2 == want["hidden_l2"]
            assert result.maximum_lower_bound == want["maximum_lower_bound"]
            assert result.candidate_count == want["candidate_count"] and result.overflow == 0
            assert result.exact_top1_token_id == want["top1_token"]
            assert result.exact_top1_logit == want["top1_logit"]
            assert torch.equal(logits.cpu(), want["logits"])    # approximate everywhere, exact at the candidates
    finally:
        head.release()


def test_lm_head_ties_and_overflow(package, oracle):
    device = torch.device("cuda", 0)
    weight = _matrix(1, SEED + 3).repeat(1500, 1).contiguous()
    head = package.LmHead(weight.to(device))
    try:
        head.launch(_hidden(SEED + 30).to(device))
        with pytest.raises(package.AimaMoeError) as error:
            head.result()
        assert error.value.status == -8
    finally:
        head.release()


def test_lm_head_full_vocabulary_agrees_with_the_exact_gemv(package):
    """248 320 rows (the reference's vocabulary): certified token == arg-max of the exact BF16 logits."""
    device = torch.device("cuda", 0)
    rows = 248320
    generator = torch.Generator(device=device).manual_seed(SEED)
    weight = (torch.randn(rows, 2048, generator=generator, device=device) * 0.02).to(torch.bfloat16)
    head = package.LmHead(weight)
    provider = package.MoeProvider(layers=1)
    try:
        for case in range(3):
            hidden = torch.randn(2048, generator=generator, device=device).to(torch.bfloat16)
            logits = head.launch(hidden)
            result = head.result()
            exact = provider.gemv(weight, hidden).float()
            best = exact.max()
            want_token = int((exact == best).nonzero()[0])
            assert result.overflow == 0 and 1 <= result.candidate_count <= 1024
            assert result.exact_top1_token_id == want_token
            assert result.exact_top1_logit == float(best)
            assert float(logits[want_token]) == float(best)
            # every approximate logit is within its bound of the exact one (BF16 rounding of the exact value included)
            assert float((logits - exact).abs().max()) < 0.05
    finally:
        provider.release()
        head.release()
