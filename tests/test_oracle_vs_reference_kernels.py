"""Pins the CPU oracle (oracle/moe_oracle.c) to the reference's OWN kernels.

oracle/build_ref.py cuts the scalar kernels of the MoE path out of the reference checkout and
compiles them for the host (oracle/_ref/libmoe_ref.so); here every oracle stage is run beside the
reference kernel it restates, on the same seeded inputs:

* bit for bit where the arithmetic is fully specified by the source: top-8 selection and tie
  order (native/src/native_moe_prefill.hip.cpp:234-323), the 8-way tree sum (:404-431), the add pair
  (native/src/native_pointwise.hip.cpp:94-107), RMSNorm incl. its summation order and the rounded
  reciprocal square root (:37-69, 109-182), the block-32 dispatch count (:325-382), and the LM-head
  row quantisation (native/src/native_lm_head.hip.cpp:53-115);
* to within one BF16 ulp on a small fraction of elements where the kernel calls expf (softmax
  weights, SiLU, sigmoid): the device library's expf is not specified bit for bit, the host build of
  the reference uses glibc's, the oracle a fixed polynomial that the CUDA kernels share.

Skipped when neither the reference checkout nor a prebuilt library is present.
"""
from __future__ import annotations

import ctypes
import sys
from ctypes import c_size_t, c_void_p
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "oracle"))
import build_ref  # noqa: E402
import moe_oracle  # noqa: E402
import ref_kernels  # noqa: E402

H, E, K, I = 2048, 256, 8, 512


@pytest.fixture(scope="module")
def ref():
    build_ref.build()
    if not ref_kernels.available():
        pytest.skip("oracle/_ref is not built and the reference checkout is absent")
    return ref_kernels.RefKernels()


@pytest.fixture(scope="module")
def oracle():
    moe_oracle.build()
    lib = moe_oracle.lib()
    for name in ("aima_or_shared_silu_mul", "aima_or_sigmoid_scale", "aima_or_expert_silu_mul", "aima_or_sum8",
                 "aima_or_add_pair", "aima_or_topk_prefill_rows"):
        getattr(lib, name).restype = None
    lib.aima_or_rsqrt.restype = ctypes.c_float
    lib.aima_or_rsqrt.argtypes = [ctypes.c_float]
    return lib


def p(array: np.ndarray) -> c_void_p:
    assert array.flags["C_CONTIGUOUS"]
    return c_void_p(array.ctypes.data)


def bf16_bits(tensor: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(tensor.to(torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16))


def normal_bits(shape, seed: int, scale: float = 1.0) -> np.ndarray:
    generator = torch.Generator().manual_seed(seed)
    return bf16_bits(torch.randn(*shape, generator=generator) * scale)


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in BF16 steps between two arrays of BF16 bit patterns of the same sign."""
    def key(bits):
        signed = bits.astype(np.int32)
        return np.where(signed & 0x8000, 0x8000 - signed, signed)
    return np.abs(key(a) - key(b))


def oracle_topk_rows(oracle, logits_bits: np.ndarray):
    tokens = logits_bits.shape[0]
    ids = np.empty((tokens, K), np.int32)
    scores = np.empty((tokens, K), np.float32)
    weights = np.empty((tokens, K), np.uint16)
    oracle.aima_or_topk_prefill_rows(p(logits_bits), ctypes.c_int(tokens), p(ids), p(scores), p(weights))
    return ids, scores, weights


@pytest.mark.parametrize("regime", ["tie_stress_eighths", "bf16_normal", "constant_rows", "two_values"])
def test_prefill_selection_and_tie_order_equal_the_reference_kernel(ref, oracle, regime):
    generator = torch.Generator().manual_seed(20260 + len(regime))
    rows = 3000
    if regime == "tie_stress_eighths":        # logits in steps of 1/8: many exact ties at the threshold
        logits = torch.round(torch.randn(rows, E, generator=generator) * 8.0) / 8.0
    elif regime == "bf16_normal":             # what the router GEMM produces: BF16-rounded N(0, 1)
        logits = torch.randn(rows, E, generator=generator)
    elif regime == "constant_rows":           # all 256 equal: selection is decided by the tie rule alone
        logits = torch.randn(rows, 1, generator=generator).expand(rows, E).contiguous()
    else:                                      # two distinct values per row, the larger on a random subset
        pick = torch.rand(rows, E, generator=generator) < torch.rand(rows, 1, generator=generator) * 0.1
        logits = torch.where(pick, torch.tensor(1.5), torch.tensor(-0.25))
    bits = bf16_bits(logits)
    ref_scores, ref_ids64, ref_ids32, ref_weights = ref.router_topk8_softmax(bits)
    ids, scores, weights = oracle_topk_rows(oracle, bits)
    assert np.array_equal(ref_ids32, ids), "expert ids or their order differ from the reference kernel"
    assert np.array_equal(ref_ids64, ids.astype(np.int64))
    assert np.array_equal(ref_scores.view(np.uint32), scores.view(np.uint32)), "selected scores differ"
    distance = ulp_distance(ref_weights, weights)
    assert distance.max() <= 1, "a softmax weight is more than one BF16 step from the reference kernel's"
    assert (distance != 0).mean() <= 2.0e-3, f"{(distance != 0).mean():.2e} of the weights differ"


def test_tree_sum_of_eight_and_add_pair_equal_the_reference_kernels(ref, oracle):
    tokens = 64
    slots = normal_bits((tokens, K, H), 11, 0.05)
    want = ref.moe_sum8(slots)
    got = np.empty((tokens, H), np.uint16)
    oracle.aima_or_sum8(p(slots), p(got), c_size_t(tokens))
    assert np.array_equal(want, got)

    left, right, resid = normal_bits((tokens, H), 12, 0.05), normal_bits((tokens, H), 13, 0.03), normal_bits((tokens, H), 14)
    want_mid, want_out = ref.add_pair(left, right, resid)
    got_mid, got_out = np.empty_like(left), np.empty_like(left)
    oracle.aima_or_add_pair(p(left), p(right), p(resid), p(got_mid), p(got_out), c_size_t(left.size))
    assert np.array_equal(want_mid, got_mid) and np.array_equal(want_out, got_out)


@pytest.mark.parametrize("scale", [1.0, 0.01, 37.0])
def test_rmsnorm_rows_equal_the_reference_kernels(ref, oracle, scale):
    rows = 600
    x = normal_bits((rows, H), 21, scale)
    residual = normal_bits((rows, H), 22, scale)
    weight = normal_bits((H,), 23, 0.02)
    want = ref.rmsnorm(x, weight)
    _, got = moe_oracle.rmsnorm(moe_oracle.bf16_tensor(x), moe_oracle.bf16_tensor(weight))
    assert np.array_equal(want, moe_oracle.bf16_numpy(got)), "RMSNorm differs from prefill_rmsnorm_2048_kernel"

    want_resid, want_norm = ref.add_rmsnorm(x, residual, weight)
    got_resid, got_norm = moe_oracle.rmsnorm(moe_oracle.bf16_tensor(x), moe_oracle.bf16_tensor(weight),
                                             residual=moe_oracle.bf16_tensor(residual))
    assert np.array_equal(want_resid, moe_oracle.bf16_numpy(got_resid))
    assert np.array_equal(want_norm, moe_oracle.bf16_numpy(got_norm)), "add + RMSNorm differs from the reference kernel"


def test_rounded_reciprocal_square_root_equals_the_reference_function(ref, oracle):
    generator = np.random.default_rng(5)
    values = np.concatenate([
        generator.uniform(1.0e-6, 4.0, 20000), generator.uniform(4.0, 4000.0, 20000),
        np.exp(generator.uniform(np.log(1.0e-12), np.log(1.0e12), 20000))]).astype(np.float32)
    differing = sum(1 for v in values if ref.rounded_rsqrt(float(v)) != float(oracle.aima_or_rsqrt(float(v))))
    assert differing == 0, f"{differing} of {values.size} values round differently"


def test_swiglu_and_sigmoid_stages_are_within_one_bf16_step_of_the_reference_kernels(ref, oracle):
    rows = 256
    gate_up = normal_bits((rows, 2 * I), 31, 1.5)
    want = ref.expert_silu_multiply(gate_up)
    got = np.empty((rows, I), np.uint16)
    oracle.aima_or_expert_silu_mul(p(gate_up), p(got), c_size_t(rows))
    distance = ulp_distance(want, got)
    assert distance.max() <= 1 and (distance != 0).mean() <= 2.0e-3

    gate, up = normal_bits((rows, I), 32, 1.5), normal_bits((rows, I), 33, 1.5)
    want = ref.shared_silu_multiply(gate, up)
    got = np.empty_like(gate)
    oracle.aima_or_shared_silu_mul(p(gate), p(up), p(got), c_size_t(gate.size))
    distance = ulp_distance(want, got)
    assert distance.max() <= 1 and (distance != 0).mean() <= 2.0e-3

    tokens = 128
    logit, down = normal_bits((tokens,), 34, 2.0), normal_bits((tokens, H), 35, 0.1)
    want = ref.shared_sigmoid_scale(logit, down)
    got = np.empty_like(down)
    oracle.aima_or_sigmoid_scale(p(logit), p(down), p(got), c_size_t(tokens))
    distance = ulp_distance(want, got)
    assert distance.max() <= 1 and (distance != 0).mean() <= 2.0e-3

    # the decode forms of the same two stages (native_pointwise.hip.cpp:184-205) on the fused 1025-wide row
    shared_input = normal_bits((1 + 2 * I,), 36, 1.5)
    want = ref.shared_activation(shared_input)
    got = np.empty(I, np.uint16)
    oracle.aima_or_shared_silu_mul(p(np.ascontiguousarray(shared_input[1:1 + I])),
                                   p(np.ascontiguousarray(shared_input[1 + I:])), p(got), c_size_t(I))
    assert ulp_distance(want, got).max() <= 1
    shared_down = normal_bits((H,), 37, 0.1)
    want = ref.shared_gate(shared_input, shared_down)
    got = np.empty(H, np.uint16)
    oracle.aima_or_sigmoid_scale(p(np.ascontiguousarray(shared_input[:1])), p(shared_down), p(got), c_size_t(1))
    assert ulp_distance(want, got).max() <= 1


def test_block32_dispatch_count_and_membership_equal_the_reference_kernel(ref, oracle):
    generator = torch.Generator().manual_seed(41)
    for tokens in (1, 7, 33, 257, 1024):
        logits = torch.randn(tokens, E, generator=generator) + torch.randn(E, generator=generator) * 2.0   # skewed
        ids = torch.topk(logits, K, dim=1).indices.to(torch.int32)
        sorted_ids, expert_ids, padded = ref.moe_align_block32(ids.numpy())
        plan = moe_oracle.dispatch_plan(ids)
        assert padded == plan["padded_rows"], "num_tokens_post_padded differs"
        # the reference fills an expert's blocks in atomic arrival order, so compare membership: the rows of
        # every 32-row block of expert e are rows the plan assigns to e, and every planned row appears once
        rows = tokens * K
        seen = np.zeros(rows, bool)
        owner = np.repeat(np.arange(E), plan["counts"].numpy())
        planned_owner = np.empty(rows, np.int64)
        planned_owner[plan["sorted_rows"].numpy()] = owner
        for block in range(padded // 32):
            expert = expert_ids[block]
            for row in sorted_ids[32 * block:32 * block + 32]:
                if row == rows:
                    continue                       # padding value
                assert planned_owner[row] == expert and not seen[row]
                seen[row] = True
        assert seen.all()


def test_lm_head_row_quantisation_equals_the_reference_kernel(ref, oracle):
    rows = 512
    source = normal_bits((rows, H), 51, 0.02)
    source[3] = 0                                  # an all-zero row takes the 1e-12 floor
    source[5, 7] = bf16_bits(torch.tensor([3.0]))[0]   # one dominant element
    want_q, want_scales, want_residual = ref.quantize_lm_head_rows(source)
    q, scales, residual = moe_oracle.lm_head_quantize(moe_oracle.bf16_tensor(source))
    assert np.array_equal(want_q, q.numpy())
    assert np.array_equal(want_scales.view(np.uint32), scales.numpy().view(np.uint32))
    assert np.array_equal(want_residual.view(np.uint32), residual.numpy().view(np.uint32))
    # the same kernel built with the multiply-add contraction a device compiler may apply
    # (value - q * scale as one fused operation): reported, the oracle follows the source as written
    fused_q, fused_scales, fused_residual = ref_kernels.RefKernels(fused=True).quantize_lm_head_rows(source)
    assert np.array_equal(fused_q, want_q) and np.array_equal(fused_scales.view(np.uint32), want_scales.view(np.uint32))
    changed = int((fused_residual.view(np.uint32) != want_residual.view(np.uint32)).sum())
    print(f"residual norms that change under contraction: {changed} of {rows}")
