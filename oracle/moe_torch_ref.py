"""torch-CPU statement of the reference's own Python MoE path (TEST INFRASTRUCTURE
ONLY: golden-vector generation, tolerance checks and the timed CPU baseline).

Each function uses the same torch operations as the reference function it
restates (benchmarks/shape-lab/four_layer_mini_engine.py):
  router_topk          :7775-7784   logits = inp @ router.t(); torch.topk(logits.float(), 8)
  routing_weights      :7786-7789   softmax(scores).to(bf16)
  expanded_routed_moe  :7791-7804   gather-per-row bmm form
  resident_routed_moe  :7904-7925   per-expert-segment form (+ build_dispatch_table :7806-7823)
  shared_expert        :8286-8303   torch branch
  layer tail           :8634-8639   after_attn + (moe_out + shared_out)
  rmsnorm              :5127-5128   torch branch with the (weight + 1) rule
torch.topk breaks ties differently from both device rules, so index parity is
never taken from here; `indices` may be supplied by the caller instead.
"""
from __future__ import annotations

from typing import Any, Mapping

import torch
import torch.nn.functional as F

TOP_K = 8
HIDDEN = 2048


def rmsnorm(inp: torch.Tensor, weight: torch.Tensor, eps: float = 1.0e-6) -> torch.Tensor:
    variance = inp.float().pow(2).mean(dim=-1, keepdim=True)
    return (inp.float() * torch.rsqrt(variance + eps) * (weight.float() + 1.0)).to(inp.dtype)


def router_topk(inp: torch.Tensor, weights: Mapping[str, Any]) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    logits = inp @ weights["router"].t()
    scores, indices = torch.topk(logits.float(), k=TOP_K, dim=-1)
    return scores, indices, logits


def routing_weights(scores: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    return torch.softmax(scores, dim=-1).to(dtype)


def expanded_routed_moe(inp: torch.Tensor, scores: torch.Tensor, indices: torch.Tensor,
                        weights: Mapping[str, Any]) -> torch.Tensor:
    """Needs weights["expert_gate_up"] [256,1024,2048] and ["expert_down"] [256,2048,512]."""
    tokens = inp.shape[0]
    dtype = inp.dtype
    expanded = inp.repeat_interleave(TOP_K, dim=0)
    flat_indices = indices.reshape(-1)
    selected_gate_up = weights["expert_gate_up"][flat_indices].transpose(1, 2)
    projected = torch.bmm(expanded.unsqueeze(1), selected_gate_up).squeeze(1)
    gate, up = projected.chunk(2, dim=-1)
    activated = (F.silu(gate.float()) * up.float()).to(dtype)
    selected_down = weights["expert_down"][flat_indices].transpose(1, 2)
    expert_out = torch.bmm(activated.unsqueeze(1), selected_down).squeeze(1)
    return (expert_out.view(tokens, TOP_K, HIDDEN) * routing_weights(scores).unsqueeze(-1)).sum(dim=1)


def build_dispatch_table(indices: torch.Tensor) -> dict[str, Any]:
    flat_indices = indices.reshape(-1)
    sorted_experts, order = torch.sort(flat_indices, stable=True)
    token_positions = torch.div(order, TOP_K, rounding_mode="floor")
    unique_experts, counts = torch.unique_consecutive(sorted_experts, return_counts=True)
    segments = []
    start = 0
    for expert_id, count in zip(unique_experts.tolist(), counts.tolist()):
        end = start + int(count)
        segments.append((int(expert_id), start, end))
        start = end
    return {"active_positions": order, "token_positions": token_positions, "segments": segments}


def resident_routed_moe(inp: torch.Tensor, scores: torch.Tensor, dispatch_table: Mapping[str, Any],
                        expert_gate_up: Any, expert_down: Any) -> torch.Tensor:
    """expert_gate_up / expert_down: indexable by expert id (tensor or dict)."""
    dtype = inp.dtype
    flat_weights = routing_weights(scores).reshape(-1)
    result = torch.zeros_like(inp)
    for expert_id, start, end in dispatch_table["segments"]:
        active_positions = dispatch_table["active_positions"][start:end]
        token_positions = dispatch_table["token_positions"][start:end]
        selected = inp[token_positions]
        projected = selected @ expert_gate_up[expert_id].t()
        gate, up = projected.chunk(2, dim=-1)
        activated = (F.silu(gate.float()) * up.float()).to(dtype)
        expert_out = activated @ expert_down[expert_id].t()
        weighted = expert_out * flat_weights[active_positions].unsqueeze(-1)
        result.index_add_(0, token_positions, weighted)
    return result


def shared_expert(inp: torch.Tensor, weights: Mapping[str, Any]) -> torch.Tensor:
    dtype = inp.dtype
    shared_gate = inp @ weights["shared_gate"].t()
    gate = inp @ weights["shared_gate_proj"].t()
    up = inp @ weights["shared_up_proj"].t()
    activated = (F.silu(gate.float()) * up.float()).to(dtype)
    shared_out = activated @ weights["shared_down_proj"].t()
    return torch.sigmoid(shared_gate).to(dtype) * shared_out


def moe_half_layer(h2: torch.Tensor, after_attn: torch.Tensor, weights: Mapping[str, Any],
                   indices: torch.Tensor | None = None, scores: torch.Tensor | None = None,
                   form: str = "expanded") -> dict[str, torch.Tensor]:
    """The MoE half of layer_body: h2, after_attn -> after_attn + (moe_out + shared_out)."""
    torch_scores, torch_indices, logits = router_topk(h2, weights)
    if indices is None:
        indices, scores = torch_indices, torch_scores
    indices = indices.to(torch.long)
    if form == "expanded":
        moe_out = expanded_routed_moe(h2, scores, indices, weights)
    else:
        gate_up = weights.get("expert_gate_up_by_id", weights.get("expert_gate_up"))
        down = weights.get("expert_down_by_id", weights.get("expert_down"))
        moe_out = resident_routed_moe(h2, scores, build_dispatch_table(indices), gate_up, down)
    shared_out = shared_expert(h2, weights)
    moe_total = moe_out + shared_out
    return {"out": after_attn + moe_total, "moe_out": moe_out, "shared_out": shared_out,
            "logits": logits, "torch_indices": torch_indices, "torch_scores": torch_scores}
