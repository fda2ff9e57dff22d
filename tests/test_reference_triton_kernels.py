"""The decode path, and the LM head with its certified top-1, against the reference's OWN Triton kernels.

tests/golden/decode_triton_<regime>.npz hold what the reference's batch-1 MoE kernels
(benchmarks/shape-lab/four_layer_mini_engine.py: triton_rmsnorm_kernel, the two-stage router top-8 with its
softmax, raw_row_gate_up_activation_kernel, raw_row_down_sum_kernel, the fused shared-expert projections)
produce on seeded inputs when they run on the CPU under Triton's interpreter
(oracle/reference_triton.py, tests/golden/make_decode_triton_golden.py).  Here the oracle -- and on a GPU the
CUDA kernel through the C ABI -- runs on the same inputs.  Bar: expert ids and their order identical (the
"ties" regimes make whole groups of experts tie exactly, inside one stage-1 block and across blocks); the
normalised input, the routing weights, the routed sum and the layer output bit-identical; the shared expert,
whose 512-term dots the reference sums in another order, identical in at least 99.5 % of its elements and
within the reference's own gate (rel-L2 <= 0.002, cosine >= 0.999) elsewhere.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import reference_triton

GOLDEN = Path(__file__).resolve().parent / "golden"
SEED = 4321
REGIMES = ("normal", "ties8", "ties4")


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _floats(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).float()


def _by_id(inputs, ids):
    pairs = {e: inputs["expert"](e) for e in ids}
    return {e: p[0] for e, p in pairs.items()}, {e: p[1] for e, p in pairs.items()}


def _check(golden, got: dict[str, torch.Tensor]) -> None:
    """got: h2, ids, scores, weights, routed, shared, out as the path under test produced them."""
    assert got["ids"].tolist() == golden["ids"].tolist()
    assert np.array_equal(_bits(got["h2"]), golden["h2"])
    assert np.array_equal(_bits(got["weights"]), golden["weights"])
    assert np.allclose(got["scores"].cpu().numpy(), golden["scores"], rtol=2.0e-6, atol=0.0)
    assert np.array_equal(_bits(got["routed"]), golden["routed"])
    assert np.array_equal(_bits(got["out"]), golden["out"])
    shared, want = _bits(got["shared"]), golden["shared_out"]
    assert (shared == want).mean() >= 0.995
    a, b = _floats(shared), _floats(want)
    assert float((a - b).norm() / b.norm()) <= 0.002
    assert float(torch.nn.functional.cosine_similarity(a, b, dim=0)) >= 0.999


@pytest.mark.parametrize("regime", REGIMES)
def test_oracle_decode_matches_the_reference_triton_kernels(oracle, regime):
    golden = np.load(GOLDEN / f"decode_triton_{regime}.npz")
    inputs = reference_triton.case_inputs(regime, SEED)
    weights = dict(inputs["small"])
    weights["expert_gate_up_by_id"], weights["expert_down_by_id"] = _by_id(inputs, [int(e) for e in golden["ids"]])
    got = oracle.decode_layer(inputs["after_attn"], oracle.OracleLayer(weights))
    got["shared"] = got["shared_scaled"]
    _check(golden, got)
    if regime != "normal":
        scores = golden["scores"]
        group = 8 if regime == "ties8" else 4
        assert all(len(set(scores[i:i + group].tolist())) == 1 for i in range(0, 8, group)), "the regime must tie"


def test_goldens_are_what_the_reference_kernels_give():
    """Runs the reference's norm and router kernels again (seconds under the interpreter; the expert kernels take
    minutes and are covered by `make_decode_triton_golden.py --check`) and compares with the committed files."""
    if not reference_triton.SOURCE.is_file():
        pytest.skip("reference checkout not present")
    pytest.importorskip("triton")
    for regime in ("normal", "ties8"):
        out = Path(os.environ.get("TMPDIR", "/tmp")) / f"aima_decode_triton_{regime}_{os.getpid()}.npz"
        subprocess.run([sys.executable, str(Path(reference_triton.__file__)), "--regime", regime, "--seed", str(SEED),
                        "--stages", "routing", "--out", str(out)], check=True,
                       env=dict(os.environ, TRITON_INTERPRET="1"), timeout=600)
        fresh, golden = np.load(out), np.load(GOLDEN / f"decode_triton_{regime}.npz")
        out.unlink()
        for name in ("h2", "ids", "scores", "weights"):
            assert np.array_equal(fresh[name], golden[name]), (regime, name)


@pytest.mark.gpu
@pytest.mark.parametrize("regime", ("normal", "ties8"))
def test_cuda_decode_matches_the_reference_triton_kernels(package, built_library, regime):
    golden = np.load(GOLDEN / f"decode_triton_{regime}.npz")
    inputs = reference_triton.case_inputs(regime, SEED)
    device = torch.device("cuda", 0)
    synth = package.synth
    # the layer holds all 256 experts; only the eight the reference selected are ever read, the rest stay zero
    layer = {name: tensor.to(device) for name, tensor in inputs["small"].items()}
    layer["expert_gate_up"] = torch.zeros(synth.EXPERTS, 2 * synth.EXPERT_INTER, synth.HIDDEN, dtype=torch.bfloat16,
                                          device=device)
    layer["expert_down"] = torch.zeros(synth.EXPERTS, synth.HIDDEN, synth.EXPERT_INTER, dtype=torch.bfloat16,
                                       device=device)
    for e in (int(e) for e in golden["ids"]):
        gate_up, down = inputs["expert"](e)
        layer["expert_gate_up"][e].copy_(gate_up)
        layer["expert_down"][e].copy_(down)
    provider = package.MoeProvider(layers=1, max_prefill_tokens=0)
    try:
        provider.bind_layer(0, layer)
        views, tensors = provider.make_debug(1, prefill=False)
        out = provider.decode_layer(inputs["after_attn"][0].to(device), 0, debug=views)
        provider.sync_metrics()
        _check(golden, {"h2": tensors["h2"][0], "ids": tensors["topk_ids"][0].cpu(), "scores": tensors["topk_scores"][0],
                        "weights": tensors["topk_weights"][0], "routed": tensors["routed"][0],
                        "shared": tensors["shared_scaled"][0], "out": out})
    finally:
        provider.release()


def test_lm_head_certificate_follows_the_reference(oracle, tmp_path):
    """The reference's quantiser (quantize_certified_lm_head), launcher and int8 scan kernel
    (triton_lm_head_rowwise_int8_gemv_kernel, under the interpreter) and the certificate arithmetic of its
    final_logits, on a 4096-row vocabulary, beside the oracle.  The reference has two statements of the row scale --
    max / 127 in this Python function, max * fl(1 / 127) in its native kernel, which the oracle follows and is
    checked against bit for bit elsewhere -- so scales may differ in the last bit and a quantised value by one on
    such rows; the scan and the certificate are therefore followed on the ORACLE's quantised rows."""
    if not reference_triton.SOURCE.is_file():
        pytest.skip("reference checkout not present")
    pytest.importorskip("triton")
    rows, seed = 4096, 777
    weight, hidden = reference_triton.lm_head_inputs(rows, seed)
    q, scales, residual = oracle.lm_head_quantize(weight)
    given = tmp_path / "quantised.npz"
    np.savez(given, q=q.numpy(), scales=scales.numpy(), residual_l2=residual.numpy())
    out = tmp_path / "reference.npz"
    subprocess.run([sys.executable, str(Path(reference_triton.__file__)), "--lm-head-rows", str(rows), "--seed", str(seed),
                    "--quantised-from", str(given), "--out", str(out)], check=True,
                   env=dict(os.environ, TRITON_INTERPRET="1"), timeout=900)
    ref = np.load(out)
    # quantiser
    assert np.abs(scales.numpy() / ref["scales"] - 1.0).max() <= 1.2e-7
    same_scale = scales.numpy() == ref["scales"]
    assert same_scale.mean() > 0.5 and np.array_equal(q.numpy()[same_scale], ref["q"][same_scale])
    assert np.abs(q.numpy().astype(np.int32) - ref["q"].astype(np.int32)).max() <= 1
    assert np.abs(residual.numpy() / ref["residual_l2"] - 1.0).max() <= 4.0e-6
    # scan + certificate
    got = oracle.lm_head_certify(weight, q, scales, residual, hidden[0])
    assert int(ref["certified"][0]) == 1 and got["status"] == 0 and got["overflow"] == 0
    assert abs(got["hidden_l2"] / float(ref["hidden_l2"][0]) - 1.0) <= 2.0e-6
    assert abs(got["maximum_lower_bound"] - float(ref["lower_max"][0])) <= 2.0e-5
    shortlist = set(ref["shortlist"].tolist())
    outside = np.array([i for i in range(rows) if i not in shortlist])
    assert np.abs(got["logits"].numpy()[outside] - ref["approximate"][outside]).max() <= 2.0e-5
    candidates = got["candidates"].tolist()
    assert set(candidates) <= shortlist                       # the oracle keeps only rows that can still win
    assert np.array_equal(got["logits"].numpy()[candidates], ref["logits"][candidates])    # exact BF16 logits
    assert got["top1_token"] == int(ref["top1"][0])
    assert got["top1_logit"] == float(ref["logits"][got["top1_token"]])


def test_fused_add_rmsnorm_follows_the_reference_kernel(oracle, tmp_path):
    """triton_prefill_fused_add_rmsnorm_kernel (the boundary between two prefill layers) under the interpreter beside
    the oracle: the BF16 residual sum bit for bit; the normalised rows bit for bit except where the two orders of the
    2048-term sum of squares meet a rounding boundary -- at most one BF16 step, on at most 0.1 % of the elements."""
    if not reference_triton.SOURCE.is_file():
        pytest.skip("reference checkout not present")
    pytest.importorskip("triton")
    rows, seed = 33, 99
    out = tmp_path / "norm.npz"
    subprocess.run([sys.executable, str(Path(reference_triton.__file__)), "--norm-rows", str(rows), "--seed", str(seed),
                    "--out", str(out)], check=True, env=dict(os.environ, TRITON_INTERPRET="1"), timeout=600)
    ref = np.load(out)
    x, residual, weight = reference_triton.norm_inputs(rows, seed)
    residual_out, norm_out = oracle.rmsnorm(x, weight, residual)
    assert np.array_equal(_bits(residual_out), ref["residual_out"])
    got, want = _bits(norm_out), ref["norm_out"]
    assert (got == want).mean() >= 0.999
    assert np.abs(got.astype(np.int32) - want.astype(np.int32)).max() <= 1        # neighbouring BF16 values


def test_oracle_chain_matches_the_reference_triton_kernels(oracle):
    """Three half-layers, each fed the previous one's output, by the reference's kernels and by the oracle.
    Teacher-forced (every layer gets the reference's input): ids in order and routing weights identical, the output
    identical except for single elements one BF16 step off (the orders of summation differ).  Free-running (the
    oracle feeds itself): the reference's own gate for such a chain, rel-L2 <= 0.02, cosine >= 0.999 and the exact
    expert set (native/src/main.cpp:1808-1815) -- here the ids stay identical in order on every layer."""
    golden = np.load(GOLDEN / "decode_triton_chain.npz")
    start = reference_triton.case_inputs("normal", SEED, 0)["after_attn"]
    assert np.array_equal(_bits(start), golden["input"])
    forced, free = start, start
    layer = 0
    while f"out{layer}" in golden.files:
        inputs = reference_triton.case_inputs("normal", SEED, layer)
        ids = [int(e) for e in golden[f"ids{layer}"]]
        weights = dict(inputs["small"])
        weights["expert_gate_up_by_id"], weights["expert_down_by_id"] = _by_id(inputs, ids)
        oracle_layer = oracle.OracleLayer(weights)
        want = golden[f"out{layer}"]
        got = oracle.decode_layer(forced, oracle_layer)
        assert got["ids"].tolist() == ids, layer
        assert np.array_equal(_bits(got["weights"]), golden[f"weights{layer}"]), layer
        out = _bits(got["out"])
        assert (out == want).mean() >= 0.999, layer
        assert np.abs(out.astype(np.int32) - want.astype(np.int32)).max() <= 1, layer
        run = oracle.decode_layer(free, oracle_layer)
        assert run["ids"].tolist() == ids, layer
        a, b = _floats(_bits(run["out"])), _floats(want)
        assert float((a - b).norm() / b.norm()) <= 0.02, layer
        assert float(torch.nn.functional.cosine_similarity(a, b, dim=0)) >= 0.999, layer
        forced = _floats(want).to(torch.bfloat16).reshape(1, -1)
        free = run["out"].reshape(1, -1)
        layer += 1
    assert layer == 3
