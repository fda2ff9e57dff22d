"""ctypes wrapper of the plain-C CPU oracle (oracle/moe_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's cpu_baseline / reference arm.  The CUDA library never uses it.
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int32, c_size_t, c_uint16, c_void_p
from pathlib import Path
from typing import Any, Mapping

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libmoe_oracle.so"

H, E, K, I, SI = 2048, 256, 8, 512, 512


class Layer(ctypes.Structure):
    _fields_ = [
        ("router", c_void_p), ("gate_up", POINTER(c_void_p)), ("down", POINTER(c_void_p)),
        ("shared_gate", c_void_p), ("shared_gate_proj", c_void_p), ("shared_up_proj", c_void_p),
        ("shared_down_proj", c_void_p), ("norm_weight", c_void_p), ("router_bias", c_void_p),
        ("router_quant_eighths", c_int32),
    ]


class Debug(ctypes.Structure):
    _fields_ = [("h2", c_void_p), ("logits", c_void_p), ("ids", c_void_p), ("scores", c_void_p),
                ("weights", c_void_p), ("shared_scaled", c_void_p), ("routed", c_void_p)]


def build(force: bool = False) -> Path:
    source = HERE / "moe_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "libmoe_oracle.so"], check=True,
                       capture_output=True)
    return LIB_PATH


_LIB = None


class LmHeadResult(ctypes.Structure):
    _fields_ = [("hidden_l2", c_float), ("maximum_lower_bound", c_float), ("exact_top1_logit", c_float),
                ("exact_top1_token_id", ctypes.c_uint32), ("candidate_count", ctypes.c_uint32),
                ("overflow", ctypes.c_uint32)]


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            build()
        _LIB = ctypes.CDLL(str(LIB_PATH))
        _LIB.aima_or_expf.restype = c_float
        _LIB.aima_or_expf.argtypes = [c_float]
        _LIB.aima_or_dot.restype = c_float
        _LIB.aima_or_dot.argtypes = [c_void_p, c_void_p, c_int]
        _LIB.aima_or_rmsnorm.restype = None
        _LIB.aima_or_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float]
        _LIB.aima_or_router_logits.restype = None
        _LIB.aima_or_router_logits.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        for name in ("aima_or_topk_prefill", "aima_or_topk_decode"):
            getattr(_LIB, name).restype = None
            getattr(_LIB, name).argtypes = [c_void_p, c_void_p, c_void_p, c_void_p]
        _LIB.aima_or_decode_layer.restype = c_int
        _LIB.aima_or_decode_layer.argtypes = [c_void_p, POINTER(Layer), c_float, c_void_p, POINTER(Debug)]
        _LIB.aima_or_prefill_layer.restype = c_int
        _LIB.aima_or_prefill_layer.argtypes = [c_void_p, c_void_p, POINTER(Layer), c_void_p, c_int,
                                               c_void_p, POINTER(Debug)]
        _LIB.aima_or_router_prefill_rows.restype = None
        _LIB.aima_or_router_prefill_rows.argtypes = [c_void_p, POINTER(Layer), c_int, c_void_p, c_void_p, c_void_p,
                                                     c_void_p]
        _LIB.aima_or_prefill_layer_forced.restype = c_int
        _LIB.aima_or_prefill_layer_forced.argtypes = [c_void_p, c_void_p, POINTER(Layer), c_void_p, c_int, c_void_p,
                                                      c_void_p, c_void_p, c_void_p, c_void_p]
        _LIB.aima_or_dispatch_plan.restype = None
        _LIB.aima_or_dispatch_plan.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
        _LIB.aima_or_gemv.restype = None
        _LIB.aima_or_gemv.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int]
        _LIB.aima_or_compare_bf16.restype = None
        _LIB.aima_or_compare_bf16.argtypes = [c_void_p, c_void_p, c_size_t, POINTER(c_double)]
        _LIB.aima_or_lm_head_quantize.restype = None
        _LIB.aima_or_lm_head_quantize.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p]
        _LIB.aima_or_lm_head_certify.restype = c_int
        _LIB.aima_or_lm_head_certify.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_void_p, POINTER(LmHeadResult), c_void_p]
    return _LIB


def _bf16_ptr(tensor: torch.Tensor | None) -> c_void_p:
    if tensor is None:
        return c_void_p(0)
    assert tensor.dtype == torch.bfloat16 and tensor.is_contiguous() and not tensor.is_cuda
    return c_void_p(tensor.data_ptr())


def bf16_numpy(tensor: torch.Tensor) -> np.ndarray:
    """BF16 tensor -> uint16 bit patterns."""
    return tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


class OracleLayer:
    """Keeps the ctypes view of one layer's CPU weights alive."""

    def __init__(self, weights: Mapping[str, Any], router_bias: torch.Tensor | None = None,
                 quant_eighths: bool = False) -> None:
        self._keep = []
        gate_up = (c_void_p * E)()
        down = (c_void_p * E)()
        by_gate_up = weights.get("expert_gate_up_by_id")
        by_down = weights.get("expert_down_by_id")
        if by_gate_up is None:
            full_gate_up = weights["expert_gate_up"].contiguous()
            full_down = weights["expert_down"].contiguous()
            self._keep += [full_gate_up, full_down]
            by_gate_up = {e: full_gate_up[e] for e in range(full_gate_up.shape[0])}
            by_down = {e: full_down[e] for e in range(full_down.shape[0])}
        for e in range(E):
            if e in by_gate_up:
                t = by_gate_up[e].contiguous()
                d = by_down[e].contiguous()
                self._keep += [t, d]
                gate_up[e] = t.data_ptr()
                down[e] = d.data_ptr()
            else:
                gate_up[e] = None
                down[e] = None
        self._gate_up, self._down = gate_up, down
        small = {}
        for name in ("router", "shared_gate", "shared_gate_proj", "shared_up_proj", "shared_down_proj",
                     "post_attention_layernorm"):
            tensor = weights.get(name)
            small[name] = None if tensor is None else tensor.contiguous()
            self._keep.append(small[name])
        self._bias = None if router_bias is None else router_bias.to(torch.float32).contiguous()
        self.c = Layer(
            _bf16_ptr(small["router"]), ctypes.cast(gate_up, POINTER(c_void_p)),
            ctypes.cast(down, POINTER(c_void_p)), _bf16_ptr(small["shared_gate"]),
            _bf16_ptr(small["shared_gate_proj"]), _bf16_ptr(small["shared_up_proj"]),
            _bf16_ptr(small["shared_down_proj"]), _bf16_ptr(small["post_attention_layernorm"]),
            c_void_p(0 if self._bias is None else self._bias.data_ptr()), int(quant_eighths))


def _debug_buffers(tokens: int) -> tuple[Debug, dict[str, torch.Tensor]]:
    t = {
        "h2": torch.zeros(tokens, H, dtype=torch.bfloat16),
        "logits": torch.zeros(tokens, E, dtype=torch.float32),
        "ids": torch.zeros(tokens, K, dtype=torch.int32),
        "scores": torch.zeros(tokens, K, dtype=torch.float32),
        "weights": torch.zeros(tokens, K, dtype=torch.bfloat16),
        "shared_scaled": torch.zeros(tokens, H, dtype=torch.bfloat16),
        "routed": torch.zeros(tokens, H, dtype=torch.bfloat16),
    }
    d = Debug(*[c_void_p(t[name].data_ptr()) for name in
                ("h2", "logits", "ids", "scores", "weights", "shared_scaled", "routed")])
    return d, t


def decode_layer(after_attn: torch.Tensor, layer: OracleLayer, eps: float = 1.0e-6) -> dict[str, torch.Tensor]:
    """after_attn: BF16 [2048] -> dict(out, h2, logits, ids, scores, weights, shared_scaled, routed)."""
    x = after_attn.reshape(H).contiguous()
    out = torch.zeros(H, dtype=torch.bfloat16)
    debug, tensors = _debug_buffers(1)
    status = lib().aima_or_decode_layer(_bf16_ptr(x), ctypes.byref(layer.c), eps, _bf16_ptr(out),
                                        ctypes.byref(debug))
    if status != 0:
        raise RuntimeError("oracle: a selected expert has no weights materialised")
    tensors = {k: v[0] for k, v in tensors.items()}
    tensors["out"] = out
    return tensors


def router_ids_decode(after_attn: torch.Tensor, layer: OracleLayer, eps: float = 1.0e-6) -> torch.Tensor:
    """Expert ids the decode path selects for one token (cheap: no expert math)."""
    x = after_attn.reshape(H).contiguous()
    h2 = torch.zeros(H, dtype=torch.bfloat16)
    lib().aima_or_rmsnorm(_bf16_ptr(x), None, layer.c.norm_weight, None, _bf16_ptr(h2), 1, eps)
    logits = torch.zeros(E, dtype=torch.float32)
    lib().aima_or_router_logits(_bf16_ptr(h2), layer.c.router, layer.c.router_bias,
                                layer.c.router_quant_eighths, c_void_p(logits.data_ptr()))
    ids = torch.zeros(K, dtype=torch.int32)
    scores = torch.zeros(K, dtype=torch.float32)
    weights = torch.zeros(K, dtype=torch.bfloat16)
    lib().aima_or_topk_decode(c_void_p(logits.data_ptr()), c_void_p(ids.data_ptr()),
                              c_void_p(scores.data_ptr()), _bf16_ptr(weights))
    return ids


def router_prefill(h2: torch.Tensor, layer: OracleLayer) -> dict[str, torch.Tensor]:
    """Prefill routing only: BF16-rounded logits, ids, scores, weights for every row of h2."""
    h2 = h2.reshape(-1, H).contiguous()
    tokens = h2.shape[0]
    logits = torch.zeros(tokens, E, dtype=torch.float32)
    ids = torch.zeros(tokens, K, dtype=torch.int32)
    scores = torch.zeros(tokens, K, dtype=torch.float32)
    weights = torch.zeros(tokens, K, dtype=torch.bfloat16)
    lib().aima_or_router_prefill_rows(_bf16_ptr(h2), ctypes.byref(layer.c), tokens, c_void_p(logits.data_ptr()),
                                      c_void_p(ids.data_ptr()), c_void_p(scores.data_ptr()), _bf16_ptr(weights))
    return {"logits": logits, "ids": ids, "scores": scores, "weights": weights}


def prefill_layer_forced(h2: torch.Tensor, residual: torch.Tensor, layer: OracleLayer, select: list[int],
                         ids: torch.Tensor, weights: torch.Tensor) -> dict[str, torch.Tensor]:
    """Expert arithmetic of the rows in `select` with the routing supplied: ids int32 [len(select), 8],
    weights BF16 [len(select), 8]."""
    h2 = h2.reshape(-1, H).contiguous()
    residual = residual.reshape(-1, H).contiguous()
    sel = torch.tensor(list(select), dtype=torch.int32)
    ids = ids.to(torch.int32).contiguous()
    weights = weights.to(torch.bfloat16).contiguous()
    assert ids.shape == (len(select), K) and weights.shape == (len(select), K)
    out = torch.zeros(len(select), H, dtype=torch.bfloat16)
    routed = torch.zeros(len(select), H, dtype=torch.bfloat16)
    shared = torch.zeros(len(select), H, dtype=torch.bfloat16)
    status = lib().aima_or_prefill_layer_forced(_bf16_ptr(h2), _bf16_ptr(residual), ctypes.byref(layer.c),
                                                c_void_p(sel.data_ptr()), len(select), c_void_p(ids.data_ptr()),
                                                _bf16_ptr(weights), _bf16_ptr(out), _bf16_ptr(routed), _bf16_ptr(shared))
    if status != 0:
        raise RuntimeError("oracle: a forced expert id is out of range or has no weights materialised")
    return {"out": out, "routed": routed, "shared_scaled": shared}


def topk_prefill(logits: torch.Tensor) -> dict[str, torch.Tensor]:
    logits = logits.to(torch.float32).reshape(-1, E).contiguous()
    tokens = logits.shape[0]
    ids = torch.zeros(tokens, K, dtype=torch.int32)
    scores = torch.zeros(tokens, K, dtype=torch.float32)
    weights = torch.zeros(tokens, K, dtype=torch.bfloat16)
    for t in range(tokens):
        lib().aima_or_topk_prefill(c_void_p(logits[t].data_ptr()), c_void_p(ids[t].data_ptr()),
                                   c_void_p(scores[t].data_ptr()), c_void_p(weights[t].data_ptr()))
    return {"ids": ids, "scores": scores, "weights": weights}


def topk_decode(logits: torch.Tensor) -> dict[str, torch.Tensor]:
    logits = logits.to(torch.float32).reshape(-1, E).contiguous()
    tokens = logits.shape[0]
    ids = torch.zeros(tokens, K, dtype=torch.int32)
    scores = torch.zeros(tokens, K, dtype=torch.float32)
    weights = torch.zeros(tokens, K, dtype=torch.bfloat16)
    for t in range(tokens):
        lib().aima_or_topk_decode(c_void_p(logits[t].data_ptr()), c_void_p(ids[t].data_ptr()),
                                  c_void_p(scores[t].data_ptr()), c_void_p(weights[t].data_ptr()))
    return {"ids": ids, "scores": scores, "weights": weights}


def prefill_layer(h2: torch.Tensor, residual: torch.Tensor, layer: OracleLayer,
                  select: list[int] | None = None) -> dict[str, torch.Tensor]:
    """Prefill half-layer for the rows in `select` (default: all).  Outputs are indexed by
    position in `select`."""
    h2 = h2.reshape(-1, H).contiguous()
    residual = residual.reshape(-1, H).contiguous()
    rows = list(range(h2.shape[0])) if select is None else list(select)
    sel = torch.tensor(rows, dtype=torch.int32)
    out = torch.zeros(len(rows), H, dtype=torch.bfloat16)
    debug, tensors = _debug_buffers(len(rows))
    status = lib().aima_or_prefill_layer(_bf16_ptr(h2), _bf16_ptr(residual), ctypes.byref(layer.c),
                                         c_void_p(sel.data_ptr()), len(rows), _bf16_ptr(out),
                                         ctypes.byref(debug))
    if status != 0:
        raise RuntimeError("oracle: a selected expert has no weights materialised")
    tensors["out"] = out
    return tensors


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None = None,
            eps: float = 1.0e-6) -> tuple[torch.Tensor | None, torch.Tensor]:
    x2 = x.reshape(-1, H).contiguous()
    rows = x2.shape[0]
    norm_out = torch.zeros_like(x2)
    residual_out = torch.zeros_like(x2) if residual is not None else None
    lib().aima_or_rmsnorm(_bf16_ptr(x2), _bf16_ptr(None if residual is None else residual.reshape(-1, H).contiguous()),
                          _bf16_ptr(weight.contiguous()), _bf16_ptr(residual_out), _bf16_ptr(norm_out),
                          rows, eps)
    return residual_out, norm_out


def dispatch_plan(ids: torch.Tensor) -> dict[str, torch.Tensor]:
    ids = ids.to(torch.int32).reshape(-1, K).contiguous()
    tokens = ids.shape[0]
    counts = torch.zeros(E, dtype=torch.int32)
    offsets = torch.zeros(E + 1, dtype=torch.int32)
    sorted_rows = torch.zeros(tokens * K, dtype=torch.int32)
    padded = torch.zeros(1, dtype=torch.int32)
    lib().aima_or_dispatch_plan(c_void_p(ids.data_ptr()), tokens, c_void_p(counts.data_ptr()),
                                c_void_p(offsets.data_ptr()), c_void_p(sorted_rows.data_ptr()),
                                c_void_p(padded.data_ptr()))
    return {"counts": counts, "offsets": offsets, "sorted_rows": sorted_rows, "padded_rows": int(padded[0])}


def gemv(weight: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    weight = weight.contiguous()
    m, k = weight.shape
    out = torch.zeros(m, dtype=torch.bfloat16)
    lib().aima_or_gemv(_bf16_ptr(weight), _bf16_ptr(x.contiguous()), _bf16_ptr(out), m, k)
    return out


def lm_head_quantize(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Row-wise int8 copy, scales and outward-rounded residual norms of a [rows, 2048] BF16 matrix."""
    weight = weight.contiguous()
    rows = weight.shape[0]
    q = torch.zeros(rows, H, dtype=torch.int8)
    scales = torch.zeros(rows, dtype=torch.float32)
    residual = torch.zeros(rows, dtype=torch.float32)
    lib().aima_or_lm_head_quantize(_bf16_ptr(weight), rows, c_void_p(q.data_ptr()), c_void_p(scales.data_ptr()),
                                   c_void_p(residual.data_ptr()))
    return q, scales, residual


def lm_head_certify(weight: torch.Tensor, q: torch.Tensor, scales: torch.Tensor, residual: torch.Tensor,
                    hidden: torch.Tensor) -> dict[str, Any]:
    """Certified top-1: approximate logits (exact at the candidates), candidates in row order, result fields."""
    weight = weight.contiguous()
    rows = weight.shape[0]
    logits = torch.zeros(rows, dtype=torch.float32)
    candidates = torch.zeros(1024, dtype=torch.int32)
    result = LmHeadResult()
    status = lib().aima_or_lm_head_certify(
        _bf16_ptr(weight), c_void_p(q.contiguous().data_ptr()), c_void_p(scales.contiguous().data_ptr()),
        c_void_p(residual.contiguous().data_ptr()), _bf16_ptr(hidden.contiguous()), rows,
        c_void_p(logits.data_ptr()), ctypes.byref(result), c_void_p(candidates.data_ptr()))
    count = min(int(result.candidate_count), 1024)
    return {"status": status, "logits": logits, "candidates": candidates[:count].clone(),
            "hidden_l2": float(result.hidden_l2), "maximum_lower_bound": float(result.maximum_lower_bound),
            "top1_logit": float(result.exact_top1_logit), "top1_token": int(result.exact_top1_token_id),
            "candidate_count": int(result.candidate_count), "overflow": int(result.overflow)}


def compare_bf16(expected: torch.Tensor, actual: torch.Tensor) -> dict[str, float]:
    """Metrics of the reference's compare_native_oracle_tensor for BF16 tensors."""
    e = expected.detach().cpu().contiguous()
    a = actual.detach().cpu().contiguous()
    assert e.shape == a.shape and e.dtype == torch.bfloat16 and a.dtype == torch.bfloat16
    result = (c_double * 5)()
    lib().aima_or_compare_bf16(_bf16_ptr(e), _bf16_ptr(a), e.numel(), result)
    return {"elements": e.numel(), "exact": int(result[0]), "max_abs": result[1], "rel_l2": result[2],
            "cosine": result[3], "finite": int(result[4])}
