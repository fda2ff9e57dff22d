"""ctypes wrapper of oracle/_ref/libmoe_ref.so: the reference's own scalar kernels for the MoE path,
compiled for the host by oracle/build_ref.py.  TEST INFRASTRUCTURE ONLY (tests, smoke check,
CPU baseline); the product never loads it.  Arrays are numpy: uint16 = BF16 bit patterns."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_size_t, c_uint, c_void_p
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
H, E, K, I = 2048, 256, 8, 512


def available() -> bool:
    return (HERE / "_ref" / "libmoe_ref.so").is_file()


class RefKernels:
    def __init__(self, fused: bool = False) -> None:
        path = HERE / "_ref" / ("libmoe_ref_fma.so" if fused else "libmoe_ref.so")
        if not path.is_file():
            raise FileNotFoundError(f"{path} is not built (python oracle/build_ref.py needs the reference checkout)")
        self.lib = ctypes.CDLL(str(path))
        self.lib.ref_rounded_rsqrtf.restype = c_float
        self.lib.ref_rounded_rsqrtf.argtypes = [c_float]

    @staticmethod
    def _p(array: np.ndarray) -> c_void_p:
        assert array.flags["C_CONTIGUOUS"]
        return c_void_p(array.ctypes.data)

    def router_topk8_softmax(self, logits: np.ndarray):
        tokens = logits.shape[0]
        assert logits.dtype == np.uint16 and logits.shape == (tokens, E)
        scores = np.empty((tokens, K), np.float32)
        ids64 = np.empty((tokens, K), np.int64)
        ids32 = np.empty((tokens, K), np.int32)
        weights = np.empty((tokens, K), np.uint16)
        self.lib.ref_router_topk8_softmax(self._p(logits), c_uint(tokens), self._p(scores), self._p(ids64),
                                          self._p(ids32), self._p(weights))
        return scores, ids64, ids32, weights

    def shared_silu_multiply(self, gate: np.ndarray, up: np.ndarray) -> np.ndarray:
        out = np.empty_like(gate)
        self.lib.ref_shared_silu_multiply(self._p(gate), self._p(up), self._p(out), c_size_t(gate.size))
        return out

    def shared_sigmoid_scale(self, gate: np.ndarray, down: np.ndarray) -> np.ndarray:
        tokens = gate.size
        assert down.shape == (tokens, H)
        out = np.empty_like(down)
        self.lib.ref_shared_sigmoid_scale(self._p(gate), self._p(down), self._p(out), c_size_t(tokens))
        return out

    def expert_silu_multiply(self, gate_up: np.ndarray) -> np.ndarray:
        rows = gate_up.shape[0]
        assert gate_up.shape == (rows, 2 * I)
        out = np.empty((rows, I), np.uint16)
        self.lib.ref_expert_silu_multiply(self._p(gate_up), self._p(out), c_size_t(rows))
        return out

    def moe_sum8(self, slots: np.ndarray) -> np.ndarray:
        tokens = slots.shape[0]
        assert slots.shape == (tokens, K, H)
        out = np.empty((tokens, H), np.uint16)
        self.lib.ref_moe_sum8(self._p(slots), self._p(out), c_uint(tokens))
        return out

    def moe_align_block32(self, topk_ids: np.ndarray):
        rows = topk_ids.size
        capacity = rows + E * 31
        sorted_ids = np.empty(capacity, np.int32)
        expert_ids = np.empty(capacity // 32, np.int32)
        padded = np.zeros(1, np.int32)
        ids = np.ascontiguousarray(topk_ids.reshape(-1).astype(np.int32))
        self.lib.ref_moe_align_block32(self._p(ids), c_size_t(rows), self._p(sorted_ids), self._p(expert_ids),
                                       self._p(padded))
        return sorted_ids, expert_ids, int(padded[0])

    def add_pair(self, left: np.ndarray, right: np.ndarray, residual: np.ndarray):
        intermediate = np.empty_like(left)
        out = np.empty_like(left)
        self.lib.ref_bf16_add_pair(self._p(left), self._p(right), self._p(residual), self._p(intermediate),
                                   self._p(out), c_size_t(left.size))
        return intermediate, out

    def rmsnorm(self, x: np.ndarray, weight: np.ndarray) -> np.ndarray:
        out = np.empty_like(x)
        self.lib.ref_rmsnorm_2048(self._p(x), self._p(weight), self._p(out), c_uint(x.shape[0]))
        return out

    def add_rmsnorm(self, x: np.ndarray, residual: np.ndarray, weight: np.ndarray):
        residual_out = np.empty_like(x)
        norm_out = np.empty_like(x)
        self.lib.ref_add_rmsnorm_2048(self._p(x), self._p(residual), self._p(weight), self._p(residual_out),
                                      self._p(norm_out), c_uint(x.shape[0]))
        return residual_out, norm_out

    def rounded_rsqrt(self, value: float) -> float:
        return float(self.lib.ref_rounded_rsqrtf(c_float(value)))

    def shared_activation(self, shared_input: np.ndarray) -> np.ndarray:
        assert shared_input.shape == (1 + 2 * I,)
        out = np.empty(I, np.uint16)
        self.lib.ref_shared_activation(self._p(shared_input), self._p(out))
        return out

    def shared_gate(self, shared_input: np.ndarray, shared_down: np.ndarray) -> np.ndarray:
        out = np.empty(H, np.uint16)
        self.lib.ref_shared_gate(self._p(shared_input), self._p(shared_down), self._p(out))
        return out

    def quantize_lm_head_rows(self, source: np.ndarray):
        rows = source.shape[0]
        assert source.shape == (rows, H) and source.dtype == np.uint16
        q = np.empty((rows, H), np.int8)
        scales = np.empty(rows, np.float32)
        residual = np.empty(rows, np.float32)
        self.lib.ref_quantize_lm_head_rows(self._p(source), c_uint(rows), self._p(q), self._p(scales), self._p(residual))
        return q, scales, residual
