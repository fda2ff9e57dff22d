"""The committed golden vectors and the torch restatement against the reference's OWN Python functions.

oracle/reference_torch.py cuts router_topk, routing_weights, expanded_routed_moe,
build_dispatch_table, resident_routed_moe, shared_expert and rmsnorm out of the reference checkout
(benchmarks/shape-lab/four_layer_mini_engine.py) and runs them on the CPU.  Skipped when the
checkout is absent (the golden files then stand for it)."""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "oracle"))
import moe_torch_ref as restated  # noqa: E402
import reference_torch  # noqa: E402

pytestmark = pytest.mark.skipif(not reference_torch.available(), reason="reference checkout absent")


def _load(name: str, path: Path):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_committed_golden_vectors_equal_the_reference_functions_output():
    generator = _load("make_golden", ROOT / "tests" / "golden" / "make_golden.py")
    for tokens in (1, 16):
        case = generator.make_case(tokens)         # also asserts restatement == reference, bit for bit
        with np.load(ROOT / "tests" / "golden" / f"config0_T{tokens}.npz") as stored:
            for key, value in case.items():
                assert np.array_equal(stored[key], value), f"T={tokens}: {key}"


def test_restated_functions_equal_the_reference_functions_on_a_ragged_batch():
    synth = _load("aima_synth", ROOT / "aima-amd395-qwen36-35b-linux-engine_b200" / "synth.py")
    torch.set_num_threads(1)
    tokens, seed, layer = 37, 77, 3
    small = synth.layer_small_weights(seed, layer)
    h2 = synth.activations(seed, tokens, "input", layer)
    reference = reference_torch.ReferenceTorch(tokens, moe_chunk_size=64)   # chunked like the engine does
    scores, indices = reference.router_topk(h2, layer, small)
    got_scores, got_indices, _ = restated.router_topk(h2, small)
    assert torch.equal(scores, got_scores) and torch.equal(indices, got_indices)
    experts = sorted(set(indices.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(experts)}
    compact = dict(small)
    compact["expert_gate_up"] = torch.stack([synth.expert_gate_up(seed, layer, e) for e in experts])
    compact["expert_down"] = torch.stack([synth.expert_down(seed, layer, e) for e in experts])
    compact_indices = torch.tensor([[remap[int(e)] for e in row] for row in indices.tolist()])
    want = reference.expanded_routed_moe(h2, scores, compact_indices, compact)
    assert torch.equal(want, restated.expanded_routed_moe(h2, scores, compact_indices, compact))
    table = reference.build_dispatch_table(compact_indices)
    want = reference.resident_routed_moe(h2, scores, table, compact, torch.zeros_like(h2))
    got = restated.resident_routed_moe(h2, scores, restated.build_dispatch_table(compact_indices),
                                       compact["expert_gate_up"], compact["expert_down"])
    assert torch.equal(want, got)
    assert torch.equal(reference.shared_expert(h2, layer, small), restated.shared_expert(h2, small))
    weight = small["post_attention_layernorm"]
    assert torch.equal(reference.rmsnorm(h2, weight), restated.rmsnorm(h2, weight))
