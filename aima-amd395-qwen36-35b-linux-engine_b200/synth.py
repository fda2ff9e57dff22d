"""Seeded synthetic weights and inputs with the shapes and value distributions
of the Qwen3.6-35B-A3B MoE layers (the real checkpoint is not redistributed).

Weights are BF16 N(0, 0.02), inputs BF16 N(0, 1).  Every tensor -- and every
expert inside the two expert tensors -- has its own torch CPU generator seed, so
a test can materialise just the experts it needs and still agree bit for bit
with a full-layer build.
"""
from __future__ import annotations

from typing import Any, Iterable

import torch

HIDDEN = 2048
EXPERTS = 256
TOP_K = 8
EXPERT_INTER = 512
SHARED_INTER = 512
WEIGHT_STD = 0.02

_TENSOR_IDS = {
    "router": 1, "shared_gate": 2, "shared_gate_proj": 3, "shared_up_proj": 4,
    "shared_down_proj": 5, "post_attention_layernorm": 6, "expert_gate_up": 7, "expert_down": 8,
    "input": 9, "residual": 10, "router_bias": 11,
}
_SHAPES = {
    "router": (EXPERTS, HIDDEN), "shared_gate": (1, HIDDEN),
    "shared_gate_proj": (SHARED_INTER, HIDDEN), "shared_up_proj": (SHARED_INTER, HIDDEN),
    "shared_down_proj": (HIDDEN, SHARED_INTER), "post_attention_layernorm": (HIDDEN,),
}


def _seed(seed: int, layer: int, name: str, index: int = 0) -> int:
    return ((seed * 128 + layer) * 16 + _TENSOR_IDS[name]) * 1024 + index


def _normal(shape: Iterable[int], seed: int, std: float) -> torch.Tensor:
    generator = torch.Generator().manual_seed(seed)
    return (torch.randn(tuple(shape), generator=generator, dtype=torch.float32) * std).to(torch.bfloat16)


def small_tensor(name: str, seed: int, layer: int) -> torch.Tensor:
    return _normal(_SHAPES[name], _seed(seed, layer, name), WEIGHT_STD)


def expert_gate_up(seed: int, layer: int, expert: int) -> torch.Tensor:
    return _normal((2 * EXPERT_INTER, HIDDEN), _seed(seed, layer, "expert_gate_up", expert), WEIGHT_STD)


def expert_down(seed: int, layer: int, expert: int) -> torch.Tensor:
    return _normal((HIDDEN, EXPERT_INTER), _seed(seed, layer, "expert_down", expert), WEIGHT_STD)


def layer_small_weights(seed: int, layer: int) -> dict[str, torch.Tensor]:
    """Everything except the two expert tensors (CPU, BF16)."""
    return {name: small_tensor(name, seed, layer) for name in _SHAPES}


def layer_weights_cpu(seed: int, layer: int, experts: Iterable[int] | None = None) -> dict[str, Any]:
    """CPU layer; `experts` limits which experts are materialised (dict e -> tensor)."""
    weights: dict[str, Any] = layer_small_weights(seed, layer)
    chosen = range(EXPERTS) if experts is None else sorted(set(int(e) for e in experts))
    weights["expert_gate_up_by_id"] = {e: expert_gate_up(seed, layer, e) for e in chosen}
    weights["expert_down_by_id"] = {e: expert_down(seed, layer, e) for e in chosen}
    return weights


def layer_weights_cuda(seed: int, layer: int, device: Any, expert_lo: int = 0,
                       expert_hi: int = EXPERTS) -> dict[str, torch.Tensor]:
    """Full layer on the GPU from the CPU generators (bit-identical to layer_weights_cpu)."""
    weights = {name: tensor.to(device) for name, tensor in layer_small_weights(seed, layer).items()}
    count = expert_hi - expert_lo
    gate_up = torch.empty(count, 2 * EXPERT_INTER, HIDDEN, dtype=torch.bfloat16, device=device)
    down = torch.empty(count, HIDDEN, EXPERT_INTER, dtype=torch.bfloat16, device=device)
    for e in range(expert_lo, expert_hi):
        gate_up[e - expert_lo].copy_(expert_gate_up(seed, layer, e))
        down[e - expert_lo].copy_(expert_down(seed, layer, e))
    weights["expert_gate_up"] = gate_up
    weights["expert_down"] = down
    return weights


def layer_weights_cuda_fast(seed: int, layer: int, device: Any, expert_lo: int = 0,
                            expert_hi: int = EXPERTS) -> dict[str, torch.Tensor]:
    """Full layer generated on the GPU (benchmark stacks: 40 layers = 64.6 GB).

    Same distributions as layer_weights_cpu but a different random stream; use
    it where no CPU copy of the weights is needed.  The expert tensors are drawn
    in blocks of 32 experts, each from its own seed, so the experts [lo, hi) a
    rank of an expert-parallel run asks for are the same values as that slice of
    the full layer.
    """
    generator = torch.Generator(device=device).manual_seed(_seed(seed, layer, "router"))

    def normal(shape: tuple[int, ...]) -> torch.Tensor:
        out = torch.empty(shape, dtype=torch.bfloat16, device=device)
        out.normal_(0.0, WEIGHT_STD, generator=generator)
        return out

    weights = {name: normal(shape) for name, shape in _SHAPES.items()}
    block = 32

    def experts(name: str, tail: tuple[int, ...]) -> torch.Tensor:
        out = torch.empty((expert_hi - expert_lo,) + tail, dtype=torch.bfloat16, device=device)
        for index in range(expert_lo // block, (expert_hi + block - 1) // block):
            block_generator = torch.Generator(device=device).manual_seed(_seed(seed, layer, name, 1 + index))
            lo, hi = max(expert_lo, index * block), min(expert_hi, (index + 1) * block)
            if hi - lo == block:
                out[lo - expert_lo:hi - expert_lo].normal_(0.0, WEIGHT_STD, generator=block_generator)
            else:
                whole = torch.empty((block,) + tail, dtype=torch.bfloat16, device=device)
                whole.normal_(0.0, WEIGHT_STD, generator=block_generator)
                out[lo - expert_lo:hi - expert_lo] = whole[lo - index * block:hi - index * block]
        return out

    weights["expert_gate_up"] = experts("expert_gate_up", (2 * EXPERT_INTER, HIDDEN))
    weights["expert_down"] = experts("expert_down", (HIDDEN, EXPERT_INTER))
    return weights


def activations(seed: int, tokens: int, name: str = "input", layer: int = 0) -> torch.Tensor:
    """BF16 N(0, 1) rows [tokens, 2048] (CPU)."""
    return _normal((tokens, HIDDEN), _seed(seed, layer, name, 0), 1.0)


def zipf_router_bias(seed: int, scale: float = 0.75, exponent: float = 1.1) -> torch.Tensor:
    """Per-expert FP32 bias that skews the tokens-per-expert histogram along a Zipf(s = exponent) ranking
    of a seeded expert permutation: bias[perm[r]] = scale * ln((r + 1) ** -exponent), centred to zero
    mean.  The logarithm makes an expert's share of the tokens, not its logit, fall with its rank; at
    8192 tokens and scale 0.75 about 16 experts get more than 1000 rows, more than 100 fewer than 10,
    some exactly one and a few none -- the histogram BASELINE config 2 describes."""
    generator = torch.Generator().manual_seed(_seed(seed, 0, "router_bias"))
    permutation = torch.randperm(EXPERTS, generator=generator)
    ranks = torch.arange(1, EXPERTS + 1, dtype=torch.float32)
    profile = scale * torch.log(ranks.pow(-exponent))
    bias = torch.empty(EXPERTS, dtype=torch.float32)
    bias[permutation] = profile
    return bias - bias.mean()


def hot_expert_bias(experts: Iterable[int], boost: float = 20.0) -> torch.Tensor:
    bias = torch.zeros(EXPERTS, dtype=torch.float32)
    bias[list(experts)] = boost
    return bias
