"""Runs the reference's OWN torch statement of the MoE half-layer on the CPU.  TEST INFRASTRUCTURE
ONLY: golden-vector generation and the check that oracle/moe_torch_ref.py restates it faithfully.

The functions are closures nested inside run_with_torch
(benchmarks/shape-lab/four_layer_mini_engine.py:2131), which needs the checkpoint to be called, so
the module cannot simply be imported and used.  Instead the `def` bodies are cut out of the
reference checkout with `ast` at run time and executed in a namespace that binds their free
variables to the values the pure-torch, CPU variant of the engine runs with (no Triton kernels,
BF16, top-8, hidden 2048).  Nothing is copied into this repository; oracle/build_ref.py saves the
cut text under oracle/_ref/ (ignored by git) for machines without the checkout.

  router_topk :7775   routing_weights :7786   expanded_routed_moe :7791   build_dispatch_table :7806
  resident_routed_moe :7904   shared_expert :8240   rmsnorm :5110
"""
from __future__ import annotations

import ast
import os
import textwrap
from pathlib import Path
from typing import Any

import torch
import torch.nn.functional as F

REFERENCE = Path(os.environ.get("AIMA_REFERENCE_ROOT", "/root/reference"))
SOURCE = REFERENCE / "benchmarks" / "shape-lab" / "four_layer_mini_engine.py"
NAMES = ("router_topk", "routing_weights", "expanded_routed_moe", "build_dispatch_table",
         "resident_routed_moe", "shared_expert", "rmsnorm")


EXTRACTED = Path(__file__).resolve().parent / "_ref" / "reference_torch_functions.py"


def available() -> bool:
    return SOURCE.is_file() or EXTRACTED.is_file()


def cut_functions() -> dict[str, tuple[str, int]]:
    """name -> (source text of the def, dedented; its line in the reference file), from the checkout."""
    text = SOURCE.read_text()
    tree = ast.parse(text)
    found: dict[str, ast.FunctionDef] = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in NAMES and node.name not in found:
            found[node.name] = node
    missing = [name for name in NAMES if name not in found]
    if missing:
        raise RuntimeError(f"reference functions not found: {missing}")
    return {name: (textwrap.dedent(" " * found[name].col_offset + ast.get_source_segment(text, found[name])),
                   found[name].lineno) for name in NAMES}


def write_extracted() -> Path | None:
    """Saves the cut functions under oracle/_ref/ (ignored by git), so that a machine without the reference
    checkout -- a GPU box timing the reference arm of the benchmark -- can still run them."""
    if not SOURCE.is_file():
        return EXTRACTED if EXTRACTED.is_file() else None
    EXTRACTED.parent.mkdir(exist_ok=True)
    pieces = ["# GENERATED from the reference checkout by oracle/reference_torch.py -- not tracked, do not edit.\n"]
    for name, (source, line) in cut_functions().items():
        pieces.append(f"# ---- {name}: benchmarks/shape-lab/four_layer_mini_engine.py:{line} ----\n{source}\n\n")
    EXTRACTED.write_text("".join(pieces))
    return EXTRACTED


class ReferenceTorch:
    """The reference's functions, bound for `tokens` rows on the CPU."""

    def __init__(self, tokens: int, moe_chunk_size: int = 1 << 30) -> None:
        never = lambda *args, **kwargs: False   # every "use the Triton kernel?" switch: no
        self.namespace: dict[str, Any] = {
            "torch": torch, "F": F, "Any": Any,
            "top_k": 8, "hidden": 2048, "shared_intermediate": 512, "tokens": tokens,
            "dtype": torch.bfloat16, "device": torch.device("cpu"), "rms_norm_eps": 1.0e-6,
            "moe_chunk_size": moe_chunk_size, "include_shared_expert": True,
            "triton_router_topk_decode": False, "torch_out_router_decode": False,
            "triton_router_topk_softmax_decode": False,
            "triton_rmsnorm_prefill": False, "triton_rmsnorm_decode": False,
            "should_use_triton_shared_expert_fused_input": never,
            "should_use_triton_shared_expert_proj": never,
            "should_use_triton_shared_expert_fused_down": never,
        }
        self.lines = {}
        if SOURCE.is_file():
            for name, (source, line) in cut_functions().items():
                exec(compile(source, f"<reference {name}>", "exec"), self.namespace)
                self.lines[name] = line
        elif EXTRACTED.is_file():
            exec(compile(EXTRACTED.read_text(), str(EXTRACTED), "exec"), self.namespace)
        else:
            raise RuntimeError("neither the reference checkout nor oracle/_ref/reference_torch_functions.py is present")

    def __getattr__(self, name: str) -> Any:
        if name in NAMES:
            return self.namespace[name]
        raise AttributeError(name)

    def moe_half_layer(self, h2: torch.Tensor, after_attn: torch.Tensor, weights: dict[str, Any],
                       form: str = "expanded") -> dict[str, torch.Tensor]:
        """layer_body's MoE tail (:8523-8639) with the reference's own functions."""
        scores, indices = self.router_topk(h2, 0, weights)
        if form == "expanded":
            moe_out = self.expanded_routed_moe(h2, scores, indices, weights)
        else:
            table = self.build_dispatch_table(indices)
            moe_out = self.resident_routed_moe(h2, scores, table, weights, torch.zeros_like(h2))
        shared_out = self.shared_expert(h2, 0, weights)
        return {"out": after_attn + (moe_out + shared_out), "moe_out": moe_out, "shared_out": shared_out,
                "scores": scores, "indices": indices, "weights": self.routing_weights(scores),
                "logits": h2 @ weights["router"].t()}
