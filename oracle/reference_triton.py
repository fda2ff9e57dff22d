"""Runs the reference's OWN Triton kernels for the batch-1 (decode) MoE half-layer on the CPU, under
Triton's interpreter (TRITON_INTERPRET=1).  TEST INFRASTRUCTURE ONLY: golden-vector generation and
the check that the oracle's decode path (oracle/moe_oracle.c) follows the kernels the reference runs.

The kernels are `@triton.jit` functions defined inside a conditional block of
benchmarks/shape-lab/four_layer_mini_engine.py, and the functions that launch them are closures of
run_with_torch (:2131), which needs the checkpoint.  The kernel definitions are therefore cut out of
the reference checkout with `ast` and written to oracle/_ref/reference_triton_kernels.py (ignored
by git; Triton reads a kernel's source from its file, so they cannot be exec'd from a string), and
launched here with the reference's own grids, block sizes and buffer dtypes:

  triton_rmsnorm_kernel :844                      launched as rmsnorm does (:5117)
  triton_router_topk_stage1_kernel :391           launched as triton_router_topk does (:7747), block_e 64, block_k 128
  triton_router_topk_stage2_kernel :426           FP32 scores
  triton_router_topk_stage2_softmax_kernel :447   BF16 routing weights
  raw_row_gate_up_activation_kernel :1152         grid (8, 512), BLOCK_H 2048, BF16 activations (:8161)
  raw_row_down_sum_kernel :1189                   grid (2048,), BLOCK_I 256, BF16 output (:8171)
  triton_matvec_kernel :304                       the fused 1025-wide shared input projection (:6096), block_n 16
  triton_fused_shared_down_kernel :360            grid (32,), block_n 64, block_k 256 (:6112)

and the tail `after_attn + (moe_out + shared_out)` of layer_body (:8634-8639) in BF16.

For the LM head with a certified top-1: triton_lm_head_rowwise_int8_gemv_kernel :1223 together with the two plain
functions around it, quantize_certified_lm_head :3553 and launch_certified_lm_head_int8 :3570, and the
certificate arithmetic of final_logits (:8656-8676), on a vocabulary small enough for the interpreter.  For the
fused residual add + RMSNorm at a prefill layer boundary: triton_prefill_fused_add_rmsnorm_kernel :862, launched as
prefill_fused_add_rmsnorm does (:5130-5149).

Nothing is copied into this repository.  Run as a script it writes one case to an .npz file:

    TRITON_INTERPRET=1 python oracle/reference_triton.py --regime normal --seed 4321 --out case.npz

Triton's interpreter narrows FP32 to BF16 by truncation where a compiled kernel rounds to nearest even; the
conversion is put right for the process before the kernels run (_round_to_nearest_even_in_the_interpreter).
"""
from __future__ import annotations

import argparse
import ast
import importlib.util
import os
import sys
import textwrap
from pathlib import Path
from typing import Any

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REFERENCE = Path(os.environ.get("AIMA_REFERENCE_ROOT", "/root/reference"))
SOURCE = REFERENCE / "benchmarks" / "shape-lab" / "four_layer_mini_engine.py"
EXTRACTED = HERE / "_ref" / "reference_triton_kernels.py"
NAMES = ("triton_matvec_kernel", "triton_fused_shared_down_kernel", "triton_router_topk_stage1_kernel",
         "triton_router_topk_stage2_kernel", "triton_router_topk_stage2_softmax_kernel", "triton_rmsnorm_kernel",
         "raw_row_gate_up_activation_kernel", "raw_row_down_sum_kernel", "triton_lm_head_rowwise_int8_gemv_kernel",
         "triton_prefill_fused_add_rmsnorm_kernel")
PLAIN = ("quantize_certified_lm_head", "launch_certified_lm_head_int8")      # ordinary functions, cut the same way

HIDDEN, EXPERTS, TOP_K, INTER = 2048, 256, 8, 512
REGIMES = ("normal", "ties8", "ties4")


def _synth() -> Any:
    spec = importlib.util.spec_from_file_location(
        "aima_synth", HERE.parent / "aima-amd395-qwen36-35b-linux-engine_b200" / "synth.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def available() -> bool:
    return SOURCE.is_file() or EXTRACTED.is_file()


def cut_kernels() -> dict[str, tuple[str, int]]:
    """name -> (source text of the def, dedented; its line in the reference file), from the checkout."""
    text = SOURCE.read_text()
    tree = ast.parse(text)
    found: dict[str, ast.FunctionDef] = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in NAMES + PLAIN and node.name not in found:
            is_kernel = any("jit" in ast.unparse(d) for d in node.decorator_list)
            if is_kernel != (node.name in NAMES):
                raise RuntimeError(f"{node.name}: Triton kernel or plain function, not what was expected")
            found[node.name] = node
    missing = [name for name in NAMES + PLAIN if name not in found]
    if missing:
        raise RuntimeError(f"reference kernels not found: {missing}")
    return {name: (textwrap.dedent(" " * found[name].col_offset + ast.get_source_segment(text, found[name])),
                   found[name].lineno) for name in NAMES + PLAIN}


def write_extracted() -> Path | None:
    """Saves the cut kernels under oracle/_ref/ (ignored by git)."""
    if not SOURCE.is_file():
        return EXTRACTED if EXTRACTED.is_file() else None
    EXTRACTED.parent.mkdir(exist_ok=True)
    pieces = ["# GENERATED from the reference checkout by oracle/reference_triton.py -- not tracked, do not edit.\n"
              "from typing import Any\n\nimport torch\nimport triton\nimport triton.language as tl\n\n"]
    for name, (source, line) in cut_kernels().items():
        pieces.append(f"# ---- {name}: benchmarks/shape-lab/four_layer_mini_engine.py:{line} ----\n"
                      f"{'@triton.jit' + chr(10) if name in NAMES else ''}{source}\n\n")
    EXTRACTED.write_text("".join(pieces))
    return EXTRACTED


def _round_to_nearest_even_in_the_interpreter() -> None:
    """Triton's interpreter narrows FP32 to BF16 by dropping the low 16 bits (its cast passes no rounding mode),
    while a compiled kernel rounds to nearest even (cvt.rn.bf16.f32), which is also what the reference's
    buffers receive on its GPU.  The interpreter's conversion routine is replaced, for this process only, by one
    that rounds FP32 -> BF16 to nearest even; every other conversion goes to the original routine."""
    import triton.language as tl
    import triton.runtime.interpreter as interpreter

    original = interpreter._convert_float
    if getattr(original, "rounds_bf16_to_nearest_even", False):
        return

    def convert(values: np.ndarray, source: Any, target: Any, rounding_mode: Any) -> np.ndarray:
        if source == tl.float32 and target == tl.bfloat16:
            as_float = np.frombuffer(values.tobytes(), dtype=np.float32).copy()
            rounded = torch.from_numpy(as_float).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
            return rounded.reshape(values.shape)
        return original(values, source, target, rounding_mode)

    convert.rounds_bf16_to_nearest_even = True
    interpreter._convert_float = convert


def load_kernels() -> Any:
    if os.environ.get("TRITON_INTERPRET") != "1":
        raise RuntimeError("set TRITON_INTERPRET=1 before Python starts: the kernels run under Triton's interpreter")
    _round_to_nearest_even_in_the_interpreter()
    if write_extracted() is None:
        raise RuntimeError("neither the reference checkout nor oracle/_ref/reference_triton_kernels.py is present")
    spec = importlib.util.spec_from_file_location("reference_triton_kernels", EXTRACTED)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


# ---------------------------------------------------------------------------------------------------
# Seeded inputs (no Triton needed: the tests rebuild them to run the oracle on the same data)
# ---------------------------------------------------------------------------------------------------
def case_inputs(regime: str, seed: int, layer: int = 0) -> dict[str, Any]:
    """The layer's small weights, the token, and a function that materialises one expert's weights.

    normal: N(0, 0.02) weights, N(0, 1) token.   ties8 / ties4: router rows shared by groups of experts, so that
    their logits are equal whatever the order of summation -- experts e with the same (e mod 64) div 2 (groups
    of eight: two neighbours in each of the four stage-1 blocks) or the same (e mod 128) div 2 (groups of four).
    The eight selected are then one or two whole groups, and both stages must break the ties to the lowest id."""
    if regime not in REGIMES:
        raise ValueError(regime)
    synth = _synth()
    small = synth.layer_small_weights(seed, layer)
    if regime != "normal":
        period = 64 if regime == "ties8" else 128
        base = small["router"]
        index = torch.tensor([(e % period) // 2 for e in range(EXPERTS)])
        small["router"] = base[index].contiguous()
    after_attn = synth.activations(seed, 1, "residual", layer)
    return {"small": small, "after_attn": after_attn,
            "expert": lambda e: (synth.expert_gate_up(seed, layer, e), synth.expert_down(seed, layer, e))}


# ---------------------------------------------------------------------------------------------------
# The reference's launch sequence
# ---------------------------------------------------------------------------------------------------
def decode_half_layer(kernels: Any, after_attn: torch.Tensor, small: dict[str, torch.Tensor], expert: Any,
                      eps: float = 1.0e-6, stages: str = "all") -> dict[str, torch.Tensor]:
    """stages = "routing": norm and router only (seconds under the interpreter; the expert kernels take a minute)."""
    import triton

    bf16 = torch.bfloat16
    x = after_attn.reshape(HIDDEN).contiguous()
    # rmsnorm (:5110-5126)
    h2 = torch.empty(1, HIDDEN, dtype=bf16)
    kernels.triton_rmsnorm_kernel[(1,)](x, small["post_attention_layernorm"], h2.reshape(HIDDEN), HIDDEN, eps,
                                        block_h=triton.next_power_of_2(HIDDEN), num_warps=8)
    inp = h2.reshape(HIDDEN)
    # triton_router_topk (:7731-7773)
    router_t = small["router"].t().contiguous()
    block_e, block_k = 64, 128
    num_blocks = triton.cdiv(EXPERTS, block_e)
    partial_values = torch.empty(num_blocks * TOP_K, dtype=torch.float32)
    partial_ids = torch.empty(num_blocks * TOP_K, dtype=torch.int32)
    kernels.triton_router_topk_stage1_kernel[(num_blocks,)](inp, router_t, partial_values, partial_ids, HIDDEN, EXPERTS,
                                                            block_e=block_e, block_k=block_k, num_warps=4)
    num_candidates = num_blocks * TOP_K
    scores = torch.empty(1, TOP_K, dtype=torch.float32)
    ids_plain = torch.empty(1, TOP_K, dtype=torch.int32)
    kernels.triton_router_topk_stage2_kernel[(1,)](partial_values, partial_ids, scores.reshape(TOP_K),
                                                   ids_plain.reshape(TOP_K), num_candidates,
                                                   block_c=triton.next_power_of_2(num_candidates), num_warps=4)
    weights = torch.empty(1, TOP_K, dtype=bf16)
    ids = torch.empty(1, TOP_K, dtype=torch.int32)
    kernels.triton_router_topk_stage2_softmax_kernel[(1,)](partial_values, partial_ids, weights.reshape(TOP_K),
                                                           ids.reshape(TOP_K), num_candidates,
                                                           block_c=triton.next_power_of_2(num_candidates), num_warps=4)
    if not torch.equal(ids, ids_plain):
        raise RuntimeError("the reference's two stage-2 kernels disagree on the ids")
    if stages == "routing":
        return {"h2": h2[0], "ids": ids[0], "scores": scores[0], "weights": weights[0]}
    # routed experts (:8119-8183).  The kernels index a dense [experts, ...] tensor by expert id; only the eight
    # selected experts are materialised here, so they are packed and addressed as experts 0..7 -- same arithmetic.
    chosen = [int(e) for e in ids.reshape(TOP_K)]
    pairs = [expert(e) for e in chosen]
    gate_up_raw = torch.stack([p[0] for p in pairs]).contiguous()
    down_raw = torch.stack([p[1] for p in pairs]).contiguous()
    packed_ids = torch.arange(TOP_K, dtype=torch.int32)
    act = torch.empty(TOP_K, INTER, dtype=bf16)
    routed = torch.empty(1, HIDDEN, dtype=bf16)
    kernels.raw_row_gate_up_activation_kernel[(TOP_K, INTER)](inp, gate_up_raw, packed_ids, act, HIDDEN, INTER,
                                                              BLOCK_H=2048, num_warps=4)
    kernels.raw_row_down_sum_kernel[(HIDDEN,)](act, down_raw, packed_ids, weights.reshape(TOP_K), routed.reshape(HIDDEN),
                                               HIDDEN, INTER, TOP_K, BLOCK_I=256, num_warps=1)
    # shared expert: fused 1025-wide input projection, fused down (:8243-8257, :6081-6123)
    fused = torch.cat([small["shared_gate"], small["shared_gate_proj"], small["shared_up_proj"]], dim=0).contiguous()
    fused_t = fused.t().contiguous()
    width = 1 + 2 * INTER
    shared_input = torch.empty(width, dtype=bf16)
    kernels.triton_matvec_kernel[(triton.cdiv(width, 16),)](inp, fused_t, shared_input, HIDDEN, width,
                                                            block_n=16, block_k=256, num_warps=2)
    shared_out = torch.empty(HIDDEN, dtype=bf16)
    kernels.triton_fused_shared_down_kernel[(triton.cdiv(HIDDEN, 64),)](
        shared_input, small["shared_down_proj"].t().contiguous(), shared_out, INTER, HIDDEN,
        block_n=64, block_k=256, num_warps=4)
    moe_out = routed + shared_out.view(1, HIDDEN)                 # :8636
    out = after_attn.view(1, HIDDEN) + moe_out                    # :8638
    return {"h2": h2[0], "ids": ids[0], "scores": scores[0], "weights": weights[0], "act": act,
            "routed": routed[0], "shared_input": shared_input, "shared_out": shared_out, "out": out[0]}


# ---------------------------------------------------------------------------------------------------
# Fused residual add + RMSNorm of a prefill layer boundary
# ---------------------------------------------------------------------------------------------------
def norm_inputs(rows: int, seed: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    synth = _synth()
    return (synth.activations(seed, rows, "input", 0), synth.activations(seed, rows, "residual", 0),
            synth.small_tensor("post_attention_layernorm", seed, 0))


def fused_add_rmsnorm(kernels: Any, x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                      eps: float = 1.0e-6) -> dict[str, torch.Tensor]:
    import triton

    rows = x.shape[0]
    residual_out = torch.empty(rows, HIDDEN, dtype=torch.bfloat16)
    norm_out = torch.empty(rows, HIDDEN, dtype=torch.bfloat16)
    kernels.triton_prefill_fused_add_rmsnorm_kernel[(rows,)](
        x.reshape(rows * HIDDEN), residual.reshape(rows * HIDDEN), weight, residual_out.reshape(rows * HIDDEN),
        norm_out.reshape(rows * HIDDEN), HIDDEN, eps, block_h=triton.next_power_of_2(HIDDEN), num_warps=8)
    return {"residual_out": residual_out, "norm_out": norm_out}


# ---------------------------------------------------------------------------------------------------
# LM head with a certified top-1
# ---------------------------------------------------------------------------------------------------
def lm_head_inputs(rows: int, seed: int) -> tuple[torch.Tensor, torch.Tensor]:
    """A [rows, 2048] BF16 N(0, 0.02) matrix and a [1, 2048] BF16 N(0, 1) final hidden state."""
    generator = torch.Generator().manual_seed(seed)
    weight = (torch.randn(rows, HIDDEN, generator=generator) * 0.02).to(torch.bfloat16)
    hidden = torch.randn(1, HIDDEN, generator=generator).to(torch.bfloat16)
    return weight, hidden


def lm_head_certified(kernels: Any, weight: torch.Tensor, final_hidden: torch.Tensor,
                      quantised: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None) -> dict[str, torch.Tensor]:
    """final_logits' certified branch (:8656-8676) with the reference's quantiser, launcher and kernel.
    `quantised` = (int8 rows, scales, residual norms) replaces the reference quantiser's output, so that the
    certificate can be followed on the very numbers another implementation quantised to."""
    q_ref, scales_ref, residual_ref = kernels.quantize_certified_lm_head(weight)
    q, scales, residual = (q_ref, scales_ref, residual_ref) if quantised is None else quantised
    logits = torch.empty(weight.shape[0], dtype=torch.float32)
    kernels.launch_certified_lm_head_int8(q, final_hidden, scales, logits)
    approximate = logits.clone()
    hidden_l2 = torch.linalg.vector_norm(final_hidden.float())
    error_bound = residual * hidden_l2
    lower_max = (logits - error_bound).max()
    upper = logits + error_bound
    upper_values, upper_indices = torch.topk(upper, k=1024)
    shortlist_weight = weight.index_select(0, upper_indices)
    exact_logits = torch.mm(final_hidden, shortlist_weight.t()).view(-1)
    certified = bool(lower_max > upper_values[-1])
    logits.scatter_(0, upper_indices, exact_logits.float())
    return {"q": q_ref, "scales": scales_ref, "residual_l2": residual_ref, "approximate": approximate,
            "hidden_l2": hidden_l2.reshape(1), "lower_max": lower_max.reshape(1), "cutoff": upper_values[-1].reshape(1),
            "shortlist": upper_indices.to(torch.int32), "logits": logits,
            "certified": torch.tensor([int(certified)], dtype=torch.int32),
            "top1": torch.argmax(logits).reshape(1).to(torch.int32)}


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def run_case(regime: str, seed: int, stages: str = "all") -> dict[str, np.ndarray]:
    kernels = load_kernels()
    inputs = case_inputs(regime, seed)
    result = decode_half_layer(kernels, inputs["after_attn"], inputs["small"], inputs["expert"], stages=stages)
    stored: dict[str, np.ndarray] = {}
    for name, tensor in result.items():
        stored[name] = bits(tensor) if tensor.dtype == torch.bfloat16 else tensor.numpy()
    return stored


def run_chain(seed: int, layers: int) -> dict[str, np.ndarray]:
    """`layers` MoE half-layers free-running: the output of layer l is the input of layer l + 1 (layer l's weights
    are the synthetic layer l of `seed`).  Stores every layer's ids, routing weights and output."""
    kernels = load_kernels()
    x = case_inputs("normal", seed, 0)["after_attn"]
    stored: dict[str, np.ndarray] = {"input": bits(x)}
    for layer in range(layers):
        inputs = case_inputs("normal", seed, layer)
        result = decode_half_layer(kernels, x, inputs["small"], inputs["expert"])
        stored[f"ids{layer}"] = result["ids"].numpy()
        stored[f"weights{layer}"] = bits(result["weights"])
        stored[f"out{layer}"] = bits(result["out"])
        x = result["out"].reshape(1, HIDDEN)
    return stored


def run_lm_head_case(rows: int, seed: int, quantised_from: str | None) -> dict[str, np.ndarray]:
    kernels = load_kernels()
    weight, hidden = lm_head_inputs(rows, seed)
    quantised = None
    if quantised_from is not None:
        given = np.load(quantised_from)
        quantised = (torch.from_numpy(given["q"]), torch.from_numpy(given["scales"]), torch.from_numpy(given["residual_l2"]))
    return {name: tensor.numpy() for name, tensor in lm_head_certified(kernels, weight, hidden, quantised).items()}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--lm-head-rows", type=int, default=0, help="run the LM-head case on this many rows instead")
    parser.add_argument("--norm-rows", type=int, default=0, help="run the fused add + RMSNorm on this many rows instead")
    parser.add_argument("--chain", type=int, default=0, help="run this many decode half-layers free-running instead")
    parser.add_argument("--quantised-from", default=None, help=".npz with q, scales, residual_l2 to certify with")
    parser.add_argument("--regime", choices=REGIMES, default="normal")
    parser.add_argument("--seed", type=int, default=4321)
    parser.add_argument("--stages", choices=("all", "routing"), default="all")
    parser.add_argument("--out", required=True)
    args = parser.parse_args()
    torch.set_num_threads(1)
    if args.chain > 0:
        np.savez_compressed(args.out, **run_chain(args.seed, args.chain))
        print(f"wrote {args.out}")
        return
    if args.norm_rows > 0:
        result = fused_add_rmsnorm(load_kernels(), *norm_inputs(args.norm_rows, args.seed))
        np.savez_compressed(args.out, **{name: bits(tensor) for name, tensor in result.items()})
        print(f"wrote {args.out}")
        return
    if args.lm_head_rows > 0:
        np.savez_compressed(args.out, **run_lm_head_case(args.lm_head_rows, args.seed, args.quantised_from))
        print(f"wrote {args.out}")
        return
    np.savez_compressed(args.out, **run_case(args.regime, args.seed, args.stages))
    print(f"wrote {args.out}")


if __name__ == "__main__":
    sys.exit(main())
