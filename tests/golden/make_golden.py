"""Generates the committed golden vectors under tests/golden/.

Runs the torch-CPU statement of the reference's Python MoE path
(oracle/moe_torch_ref.py, which restates
benchmarks/shape-lab/four_layer_mini_engine.py:7775-7804, 8286-8303, 8634-8639)
on the seeded synthetic layer of BASELINE config 0 (T in {1, 16}) and stores
its results.  The reference module itself cannot be imported: its functions are
closures inside run_with_torch (:2131) and need the 67 GB checkpoint, so this
script is the pinned stand-in; rerun it with

    python tests/golden/make_golden.py

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
    scores, indices, logits = ref.router_topk(h2, small)
    experts = sorted(set(indices.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(experts)}
    compact = dict(small)
    compact["expert_gate_up"] = torch.stack([synth.expert_gate_up(SEED, LAYER, e) for e in experts])
    compact["expert_down"] = torch.stack([synth.expert_down(SEED, LAYER, e) for e in experts])
    compact_indices = torch.tensor([[remap[int(e)] for e in row] for row in indices.tolist()])
    moe_out = ref.expanded_routed_moe(h2, scores, compact_indices, compact)
    shared_out = ref.shared_expert(h2, small)
    out = after_attn + (moe_out + shared_out)
    return {
        "seed": np.array([SEED, LAYER, tokens]),
        "logits": bits(logits), "topk_indices": indices.numpy(), "topk_scores": scores.numpy(),
        "weights": bits(ref.routing_weights(scores)), "moe_out": bits(moe_out),
        "shared_out": bits(shared_out), "out": bits(out),
    }


def main() -> None:
    here = Path(__file__).resolve().parent
    for tokens in (1, 16):
        case = make_case(tokens)
        np.savez_compressed(here / f"config0_T{tokens}.npz", **case)
        print(f"wrote config0_T{tokens}.npz", {k: v.shape for k, v in case.items()})


if __name__ == "__main__":
    main()
