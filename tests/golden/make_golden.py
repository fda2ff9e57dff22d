"""Generates the committed golden vectors under tests/golden/ from the reference's OWN code.

The reference's torch functions for the MoE half-layer (router_topk, routing_weights,
expanded_routed_moe, shared_expert; benchmarks/shape-lab/four_layer_mini_engine.py:7775-7804,
8240-8303, 8634-8639) are closures inside run_with_torch (:2131), which needs the 67 GB checkpoint to
be called; oracle/reference_torch.py cuts their `def` bodies out of the reference checkout with
`ast` and executes them with their free variables bound to the pure-torch CPU configuration.  This
script runs THOSE functions on the seeded synthetic layer of BASELINE config 0 (T in {1, 16}),
checks that the hand restatement oracle/moe_torch_ref.py gives the same bits, and stores the
results.  It needs the reference checkout (its location: AIMA_REFERENCE_ROOT in the environment):

    python tests/golden/make_golden.py            # regenerate
    python tests/golden/make_golden.py --check    # regenerate in memory and compare with the files

Stored per case (npz, BF16 as uint16 bit patterns):
  logits       [T,256]  inp @ router.t()           (BF16)
  topk_indices [T,8]    torch.topk indices          (int64; informational tie order)
  topk_scores  [T,8]    torch.topk values           (FP32)
  weights      [T,8]    softmax(scores).to(bf16)
  moe_out      [T,2048] expanded_routed_moe
  shared_out   [T,2048] shared_expert
  out          [T,2048] after_attn + (moe_out + shared_out)
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT / "oracle"))
import moe_torch_ref as ref  # noqa: E402
import reference_torch  # noqa: E402

_spec = importlib.util.spec_from_file_location(
    "aima_synth", ROOT / "aima-amd395-qwen36-35b-linux-engine_b200" / "synth.py")
synth = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(synth)

SEED = 1234
LAYER = 0


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def make_case(tokens: int) -> dict[str, np.ndarray]:
    torch.set_num_threads(1)  # fixed reduction order inside torch's BF16 matmuls
    small = synth.layer_small_weights(SEED, LAYER)
    h2 = synth.activations(SEED, tokens, "input", LAYER)
    after_attn = synth.activations(SEED, tokens, "residual", LAYER)
    reference = reference_torch.ReferenceTorch(tokens)
    scores, indices = reference.router_topk(h2, LAYER, small)
    logits = h2 @ small["router"].t()
    restated_scores, restated_indices, restated_logits = ref.router_topk(h2, small)
    assert torch.equal(scores, restated_scores) and torch.equal(indices, restated_indices)
    experts = sorted(set(indices.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(experts)}
    compact = dict(small)
    compact["expert_gate_up"] = torch.stack([synth.expert_gate_up(SEED, LAYER, e) for e in experts])
    compact["expert_down"] = torch.stack([synth.expert_down(SEED, LAYER, e) for e in experts])
    compact_indices = torch.tensor([[remap[int(e)] for e in row] for row in indices.tolist()])
    moe_out = reference.expanded_routed_moe(h2, scores, compact_indices, compact)
    shared_out = reference.shared_expert(h2, LAYER, small)
    out = after_attn + (moe_out + shared_out)
    # the hand restatement used by the tests and the CPU baseline must give the same bits
    assert torch.equal(moe_out, ref.expanded_routed_moe(h2, scores, compact_indices, compact))
    assert torch.equal(shared_out, ref.shared_expert(h2, small))
    assert torch.equal(reference.routing_weights(scores), ref.routing_weights(scores))
    table = reference.build_dispatch_table(compact_indices)
    segment_form = reference.resident_routed_moe(h2, scores, table, compact, torch.zeros_like(h2))
    assert torch.equal(segment_form, ref.resident_routed_moe(h2, scores, ref.build_dispatch_table(compact_indices),
                                                             compact["expert_gate_up"], compact["expert_down"]))
    return {
        "seed": np.array([SEED, LAYER, tokens]),
        "logits": bits(logits), "topk_indices": indices.numpy(), "topk_scores": scores.numpy(),
        "weights": bits(reference.routing_weights(scores)), "moe_out": bits(moe_out),
        "shared_out": bits(shared_out), "out": bits(out),
    }


def main() -> None:
    here = Path(__file__).resolve().parent
    check = "--check" in sys.argv
    for tokens in (1, 16):
        case = make_case(tokens)
        path = here / f"config0_T{tokens}.npz"
        if check:
            with np.load(path) as stored:
                for key, value in case.items():
                    assert np.array_equal(stored[key], value), f"{path.name}: {key} differs from the reference's output"
            print(f"{path.name}: equal to the reference's own functions")
        else:
            np.savez_compressed(path, **case)
            print(f"wrote {path.name}", {k: v.shape for k, v in case.items()})


if __name__ == "__main__":
    main()
