"""ctypes binding of the C ABI in include/aima_moe.h and a provider object with
the call shape of the reference's Python drop-in point.

The reference loads native providers with ``ctypes.CDLL(path, RTLD_LOCAL)``,
passes tensors as ``c_void_p(tensor.data_ptr())`` and the stream as
``c_void_p(torch.cuda.current_stream().cuda_stream)``
(benchmarks/shape-lab/q8192_compound_provider.py:59-66, 132-141), and calls
``launch_selected_moe(post_attention=h2, residual_hidden=after_attn,
weights=<dict of tensors>, model_layer=<int>) -> hidden``
(benchmarks/shape-lab/four_layer_mini_engine.py:8491-8502; the stub that
raises "not admitted" is q8192_compound_provider.py:388-389).  MoeProvider
keeps that signature.

There is no CPU fallback: if the shared library is missing or no sm_100 device
is present, construction fails loudly.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_uint32, c_uint64, c_void_p
from pathlib import Path
from typing import Any, Mapping

HIDDEN = 2048
EXPERTS = 256
TOP_K = 8
EXPERT_INTER = 512
SHARED_INTER = 512
MAX_LAYERS = 64

_LIB_NAME = "libaima_moe_b200.so"


class AimaMoeError(RuntimeError):
    def __init__(self, status: int, message: str) -> None:
        super().__init__(f"aima_moe status {status}: {message}")
        self.status = status


class Config(ctypes.Structure):
    _fields_ = [
        ("struct_bytes", c_uint32), ("hidden", c_uint32), ("experts", c_uint32),
        ("top_k", c_uint32), ("expert_inter", c_uint32), ("shared_inter", c_uint32),
        ("layers", c_uint32), ("max_prefill_tokens", c_uint32), ("world", c_uint32),
        ("rank", c_uint32), ("rms_eps", c_float), ("flags", c_uint32),
    ]


class LayerWeights(ctypes.Structure):
    _fields_ = [
        ("struct_bytes", c_uint32), ("reserved", c_uint32),
        ("router", c_void_p), ("router_bytes", c_uint64),
        ("expert_gate_up", c_void_p), ("expert_gate_up_bytes", c_uint64),
        ("expert_down", c_void_p), ("expert_down_bytes", c_uint64),
        ("shared_expert_gate", c_void_p), ("shared_expert_gate_bytes", c_uint64),
        ("shared_gate_proj", c_void_p), ("shared_gate_proj_bytes", c_uint64),
        ("shared_up_proj", c_void_p), ("shared_up_proj_bytes", c_uint64),
        ("shared_down_proj", c_void_p), ("shared_down_proj_bytes", c_uint64),
        ("post_attention_norm", c_void_p), ("post_attention_norm_bytes", c_uint64),
    ]


class DebugViews(ctypes.Structure):
    _fields_ = [
        ("struct_bytes", c_uint32), ("reserved", c_uint32),
        ("h2", c_void_p), ("router_logits", c_void_p), ("topk_ids", c_void_p),
        ("topk_scores", c_void_p), ("topk_weights", c_void_p), ("shared_scaled", c_void_p),
        ("routed", c_void_p), ("expert_counts", c_void_p), ("expert_offsets", c_void_p),
        ("sorted_rows", c_void_p), ("slot_dots", c_void_p), ("slot_rows", c_void_p),
    ]


class Metrics(ctypes.Structure):
    _fields_ = [
        ("struct_bytes", c_uint32), ("reserved", c_uint32),
        ("prefill_calls", c_uint64), ("decode_calls", c_uint64), ("kernel_launches", c_uint64),
        ("workspace_bytes", c_uint64), ("derived_weight_bytes", c_uint64),
        ("last_padded_routed_rows", c_int32), ("device_status", c_int32),
        ("router_candidates", c_uint64), ("router_tokens", c_uint64),
        ("router_bound_violations", c_uint64), ("router_audited_tokens", c_uint64),
        ("router_audit_mismatches", c_uint64),
    ]


class SafetensorsEntry(ctypes.Structure):
    _fields_ = [
        ("name", ctypes.c_char * 200), ("dtype", ctypes.c_char * 8), ("rank", c_uint32), ("reserved", c_uint32),
        ("shape", c_uint64 * 4), ("data_begin", c_uint64), ("data_end", c_uint64),
    ]


class ImageIngestResult(ctypes.Structure):
    _fields_ = [
        ("bytes", c_uint64), ("read_ms", ctypes.c_double), ("checksum_ms", c_float), ("direct_io", c_uint32),
        ("xor_value", c_uint64), ("sum_value", c_uint64),
    ]


class LmHeadResult(ctypes.Structure):
    _fields_ = [
        ("hidden_l2", c_float), ("maximum_lower_bound", c_float), ("exact_top1_logit", c_float),
        ("exact_top1_token_id", c_uint32), ("candidate_count", c_uint32), ("overflow", c_uint32),
    ]


# every symbol include/aima_moe.h declares: (name, restype, argtypes)
EXPORTS = [
    ("aima_moe_abi_version", c_uint32, []),
    ("aima_moe_last_error_string", c_char_p, []),
    ("aima_moe_query_workspace", c_int, [ctypes.POINTER(Config), ctypes.POINTER(c_uint64)]),
    ("aima_moe_prepare", c_int, [ctypes.POINTER(Config), ctypes.POINTER(c_void_p)]),
    ("aima_moe_bind_layer", c_int, [c_void_p, c_uint32, ctypes.POINTER(LayerWeights)]),
    ("aima_moe_set_router_hooks", c_int, [c_void_p, c_void_p, c_int]),
    ("aima_moe_prefill_launch", c_int,
     [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_uint32, ctypes.POINTER(DebugViews), c_void_p]),
    ("aima_moe_decode_launch", c_int,
     [c_void_p, c_uint32, c_void_p, c_void_p, ctypes.POINTER(DebugViews), c_void_p]),
    ("aima_moe_decode_stack_launch", c_int, [c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p]),
    ("aima_moe_prefill_stack_launch", c_int,
     [c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_uint32, c_void_p]),
    ("aima_moe_prefill_fused_launch", c_int,
     [c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_void_p]),
    ("aima_moe_rmsnorm_launch", c_int,
     [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_float, c_void_p]),
    ("aima_moe_gemv_bf16_launch", c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_void_p]),
    ("aima_moe_gemm_bf16_launch", c_int,
     [c_void_p, c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32, c_void_p]),
    ("aima_moe_decode_layers_noalloc", c_int,
     [ctypes.POINTER(LayerWeights), c_uint32, c_void_p, c_void_p, c_float, c_void_p, c_void_p]),
    ("aima_moe_ep_local_buffer", c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_uint64)]),
    ("aima_moe_ep_export", c_int, [c_void_p, c_void_p]),
    ("aima_moe_ep_connect", c_int, [c_void_p, c_uint32, c_void_p, c_void_p]),
    ("aima_moe_read_ep_prefill_stages", c_int,
     [c_void_p, ctypes.POINTER(c_float), c_uint32, ctypes.POINTER(c_uint32)]),
    ("aima_moe_set_forced_routing", c_int, [c_void_p, c_void_p, c_void_p, c_uint32]),
    ("aima_moe_set_tracing", c_int, [c_void_p, c_int]),
    ("aima_moe_debug_set_decode_epoch", c_int, [c_void_p, c_uint32]),
    ("aima_moe_read_decode_timeline", c_int,
     [c_void_p, ctypes.POINTER(c_uint64), c_uint32, ctypes.POINTER(c_uint32)]),
    ("aima_moe_read_decode_block_timelines", c_int,
     [c_void_p, ctypes.POINTER(c_uint64), c_uint32, ctypes.POINTER(c_uint32), ctypes.POINTER(c_uint32)]),
    ("aima_moe_lm_head_build", c_int, [c_void_p, c_uint32, ctypes.POINTER(c_void_p), c_void_p]),
    ("aima_moe_lm_head_views", c_int,
     [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p)]),
    ("aima_moe_lm_head_launch", c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    ("aima_moe_lm_head_read_result", c_int, [c_void_p, ctypes.POINTER(LmHeadResult)]),
    ("aima_moe_lm_head_release", c_int, [c_void_p]),
    ("aima_moe_safetensors_index", c_int,
     [ctypes.c_char_p, ctypes.POINTER(SafetensorsEntry), c_uint64, ctypes.POINTER(c_uint64)]),
    ("aima_moe_image_build_from_files", c_int,
     [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(c_uint64),
      ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint32), ctypes.POINTER(c_uint64), c_uint64,
      ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint64)]),
    ("aima_moe_image_plan", c_int,
     [ctypes.POINTER(c_uint64), ctypes.POINTER(ctypes.c_char_p), c_uint64, ctypes.POINTER(c_uint32),
      ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint64)]),
    ("aima_moe_image_checksum_host", c_int, [c_void_p, c_uint64, ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint64)]),
    ("aima_moe_image_build", c_int,
     [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint32),
      ctypes.POINTER(c_uint64), c_uint64, ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint64),
      ctypes.POINTER(c_uint64)]),
    ("aima_moe_image_scatter_ingest", c_int,
     [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint64), ctypes.POINTER(c_uint64),
      c_uint64, c_uint64, c_uint64, c_uint64, c_int, c_uint64, c_uint64, ctypes.POINTER(ImageIngestResult)]),
    ("aima_moe_sync_metrics", c_int, [c_void_p, ctypes.POINTER(Metrics)]),
    ("aima_moe_release", c_int, [c_void_p]),
]


def library_path() -> Path:
    return Path(__file__).resolve().parent / _LIB_NAME


class MoeLibrary:
    """The loaded shared library with typed entry points."""

    def __init__(self, path: Path | None = None) -> None:
        path = Path(path) if path is not None else library_path()
        if not path.is_file():
            raise FileNotFoundError(
                f"{path} is missing: build it with aima-amd395-qwen36-35b-linux-engine_b200/build.py; "
                "there is no CPU or PyTorch fallback for this path")
        self.path = path
        self.cdll = ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL)
        for name, restype, argtypes in EXPORTS:
            function = getattr(self.cdll, name)
            function.restype = restype
            function.argtypes = argtypes
            setattr(self, name, function)

    def check(self, status: int) -> None:
        if status != 0:
            message = self.aima_moe_last_error_string() or b""
            raise AimaMoeError(status, message.decode("utf-8", "replace"))


_LIBRARY: MoeLibrary | None = None


def load_library() -> MoeLibrary:
    global _LIBRARY
    if _LIBRARY is None:
        _LIBRARY = MoeLibrary()
    return _LIBRARY


def _ptr(tensor: Any) -> c_void_p:
    if tensor is None:
        return c_void_p(0)
    if not tensor.is_cuda or not tensor.is_contiguous():
        raise RuntimeError("aima_moe tensors must be contiguous CUDA tensors")
    return c_void_p(int(tensor.data_ptr()))


def _nbytes(tensor: Any) -> int:
    return 0 if tensor is None else int(tensor.numel() * tensor.element_size())


def _stream(torch: Any) -> c_void_p:
    return c_void_p(int(torch.cuda.current_stream().cuda_stream))


# reference weight-dict keys (four_layer_mini_engine.py: weights["router"],
# ["expert_gate_up"], ["expert_down"], ["shared_gate"], ["shared_gate_proj"],
# ["shared_up_proj"], ["shared_down_proj"], ["post_attention_layernorm"])
WEIGHT_KEYS = ("router", "expert_gate_up", "expert_down", "shared_gate", "shared_gate_proj",
               "shared_up_proj", "shared_down_proj")


NOALLOC_MAX_LAYERS = 8
FLAG_SIMT_PRODUCTS = 1
FLAG_EXACT_ROUTER = 2
FLAG_MATERIALIZED_DISPATCH = 8
FLAG_EP_PIPELINE_2 = 32
FLAG_EP_PIPELINE_4 = 64
FLAG_NO_DECODE_PREDICTION = 128
FLAG_AUDIT_ROUTER = 256
FLAG_TWO_SM_PRODUCTS = 512


def layer_weights_struct(weights: Mapping[str, Any]) -> LayerWeights:
    """Fills the C struct from a reference-style weight dict of CUDA tensors."""
    w = LayerWeights()
    w.struct_bytes = ctypes.sizeof(LayerWeights)
    fields = {
        "router": weights["router"], "expert_gate_up": weights["expert_gate_up"],
        "expert_down": weights["expert_down"], "shared_expert_gate": weights["shared_gate"],
        "shared_gate_proj": weights["shared_gate_proj"], "shared_up_proj": weights["shared_up_proj"],
        "shared_down_proj": weights["shared_down_proj"],
        "post_attention_norm": weights.get("post_attention_layernorm"),
    }
    for name, tensor in fields.items():
        setattr(w, name, _ptr(tensor))
        setattr(w, name + "_bytes", _nbytes(tensor))
    return w


def decode_layers_noalloc(layer_dicts: list, x_in: Any, x_out: Any, rms_eps: float = 1.0e-6,
                          device_status: Any = None, library: MoeLibrary | None = None) -> Any:
    """Calls the allocation-free decode entry point for a host that must not allocate device
    memory: no handle, the kernel's scratch is the library's static device array.  x_in / x_out
    are BF16 [2048] CUDA tensors, layer_dicts the per-layer weight dicts (at most 8)."""
    import torch

    lib = library or load_library()
    array = (LayerWeights * len(layer_dicts))(*[layer_weights_struct(w) for w in layer_dicts])
    lib.check(lib.aima_moe_decode_layers_noalloc(
        array, len(layer_dicts), _ptr(x_in), _ptr(x_out), rms_eps, _ptr(device_status), _stream(torch)))
    return x_out


def exchange_ipc_handles(mine: bytes, rank: int, world: int, group: Any = None) -> list[bytes]:
    """All-gathers one 64-byte handle per rank over torch.distributed; returns them by rank."""
    import torch
    import torch.distributed as dist

    assert len(mine) == 64
    backend = dist.get_backend(group)
    device = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    local = torch.tensor(list(mine), dtype=torch.uint8, device=device)
    gathered = [torch.empty(64, dtype=torch.uint8, device=device) for _ in range(world)]
    dist.all_gather(gathered, local, group=group)
    handles = [bytes(t.cpu().tolist()) for t in gathered]
    assert handles[rank] == mine
    return handles


class MoeProvider:
    """Owns one aima_moe handle on the current CUDA device."""

    def __init__(self, layers: int, max_prefill_tokens: int = 0, world: int = 1, rank: int = 0,
                 rms_eps: float = 1.0e-6, library: MoeLibrary | None = None, flags: int = 0) -> None:
        import torch  # device memory and streams only

        if not torch.cuda.is_available():
            raise RuntimeError("aima_moe needs a CUDA device (sm_100a); there is no CPU fallback")
        self._torch = torch
        self.lib = library or load_library()
        self.layers = layers
        self.max_prefill_tokens = max_prefill_tokens
        self.config = Config(ctypes.sizeof(Config), HIDDEN, EXPERTS, TOP_K, EXPERT_INTER, SHARED_INTER,
                             layers, max_prefill_tokens, world, rank, rms_eps, flags)
        handle = c_void_p()
        self.lib.check(self.lib.aima_moe_prepare(ctypes.byref(self.config), ctypes.byref(handle)))
        self.handle = handle
        self._keepalive: dict[int, Mapping[str, Any]] = {}
        self._hook_bias = None
        self.calls = {"selected_moe": 0, "decode": 0}

    # -- setup ---------------------------------------------------------------
    def bind_layer(self, layer: int, weights: Mapping[str, Any]) -> None:
        w = LayerWeights()
        w.struct_bytes = ctypes.sizeof(LayerWeights)
        fields = {
            "router": weights["router"], "expert_gate_up": weights["expert_gate_up"],
            "expert_down": weights["expert_down"], "shared_expert_gate": weights["shared_gate"],
            "shared_gate_proj": weights["shared_gate_proj"], "shared_up_proj": weights["shared_up_proj"],
            "shared_down_proj": weights["shared_down_proj"],
            "post_attention_norm": weights.get("post_attention_layernorm"),
        }
        for name, tensor in fields.items():
            setattr(w, name, _ptr(tensor))
            setattr(w, name + "_bytes", _nbytes(tensor))
        self.lib.check(self.lib.aima_moe_bind_layer(self.handle, layer, ctypes.byref(w)))
        self._keepalive[layer] = dict(weights)

    def set_router_hooks(self, bias: Any = None, quantize_eighths: bool = False) -> None:
        self._hook_bias = bias
        self.lib.check(self.lib.aima_moe_set_router_hooks(self.handle, _ptr(bias), int(quantize_eighths)))

    def set_forced_routing(self, ids: Any = None, weights: Any = None) -> None:
        """Qualification: int32 [T, 8] expert ids and BF16 [T, 8] weights used by the next single-layer
        prefill calls of T tokens instead of the router's; None clears."""
        self._forced = (ids, weights)          # keep the device tensors alive while set
        tokens = 0 if ids is None else int(ids.shape[0])
        self.lib.check(self.lib.aima_moe_set_forced_routing(self.handle, _ptr(ids), _ptr(weights), tokens))

    # -- debug views ---------------------------------------------------------
    def make_debug(self, tokens: int, prefill: bool, with_logits: bool = True,
                   with_slot_rows: bool = False) -> tuple[DebugViews, dict[str, Any]]:
        torch = self._torch
        dev = torch.device("cuda", torch.cuda.current_device())
        t = {
            "h2": torch.empty(tokens, HIDDEN, dtype=torch.bfloat16, device=dev),
            "router_logits": torch.empty(tokens, EXPERTS, dtype=torch.float32, device=dev),
            "topk_ids": torch.empty(tokens, TOP_K, dtype=torch.int32, device=dev),
            "topk_scores": torch.empty(tokens, TOP_K, dtype=torch.float32, device=dev),
            "topk_weights": torch.empty(tokens, TOP_K, dtype=torch.bfloat16, device=dev),
            "shared_scaled": torch.empty(tokens, HIDDEN, dtype=torch.bfloat16, device=dev),
            "routed": torch.empty(tokens, HIDDEN, dtype=torch.bfloat16, device=dev),
        }
        if not prefill:
            t["slot_dots"] = torch.zeros(TOP_K, HIDDEN, dtype=torch.float32, device=dev)
        if prefill:
            t["expert_counts"] = torch.empty(EXPERTS, dtype=torch.int32, device=dev)
            t["expert_offsets"] = torch.empty(EXPERTS + 1, dtype=torch.int32, device=dev)
            t["sorted_rows"] = torch.empty(tokens * TOP_K, dtype=torch.int32, device=dev)
        if prefill and with_slot_rows:
            t["slot_rows"] = torch.empty(tokens * TOP_K, HIDDEN, dtype=torch.bfloat16, device=dev)
        if not with_logits:
            del t["router_logits"]      # prefill then runs the production (certified) router
        views = DebugViews()
        views.struct_bytes = ctypes.sizeof(DebugViews)
        for name, tensor in t.items():
            setattr(views, name, _ptr(tensor))
        return views, t

    # -- launches ------------------------------------------------------------
    def launch_selected_moe(self, *, post_attention: Any, residual_hidden: Any,
                            weights: Mapping[str, Any] | None = None, model_layer: int,
                            out: Any = None, debug: DebugViews | None = None) -> Any:
        """Prefill MoE half of `model_layer`: h2, after_attn -> next hidden [T, 2048]."""
        torch = self._torch
        if weights is not None and model_layer not in self._keepalive:
            self.bind_layer(model_layer, weights)
        tokens = int(post_attention.shape[0])
        if out is None:
            out = torch.empty_like(residual_hidden)
        self.lib.check(self.lib.aima_moe_prefill_launch(
            self.handle, model_layer, _ptr(post_attention), _ptr(residual_hidden), _ptr(out), tokens,
            ctypes.byref(debug) if debug is not None else None, _stream(torch)))
        self.calls["selected_moe"] += 1
        return out

    def decode_layer(self, after_attn: Any, model_layer: int, out: Any = None,
                     debug: DebugViews | None = None) -> Any:
        torch = self._torch
        if out is None:
            out = torch.empty_like(after_attn)
        self.lib.check(self.lib.aima_moe_decode_launch(
            self.handle, model_layer, _ptr(after_attn), _ptr(out),
            ctypes.byref(debug) if debug is not None else None, _stream(torch)))
        self.calls["decode"] += 1
        return out

    def decode_stack(self, x_in: Any, x_out: Any, first_layer: int = 0, n_layers: int | None = None) -> Any:
        torch = self._torch
        n = self.layers - first_layer if n_layers is None else n_layers
        self.lib.check(self.lib.aima_moe_decode_stack_launch(
            self.handle, first_layer, n, _ptr(x_in), _ptr(x_out), _stream(torch)))
        self.calls["decode"] += n
        return x_out

    def prefill_stack(self, x_in: Any, x_out: Any, first_layer: int = 0, n_layers: int | None = None) -> Any:
        torch = self._torch
        n = self.layers - first_layer if n_layers is None else n_layers
        self.lib.check(self.lib.aima_moe_prefill_stack_launch(
            self.handle, first_layer, n, _ptr(x_in), _ptr(x_out), int(x_in.shape[0]), _stream(torch)))
        return x_out

    def prefill_fused(self, attn_out: Any, residual_in: Any, model_layer: int,
                      next_norm_weight: Any = None) -> tuple[Any, Any]:
        """add + RMSNorm -> MoE half -> (optional) next layer's input norm; returns (layer_out, next_norm_out)."""
        torch = self._torch
        layer_out = torch.empty_like(residual_in)
        next_norm_out = torch.empty_like(residual_in) if next_norm_weight is not None else None
        self.lib.check(self.lib.aima_moe_prefill_fused_launch(
            self.handle, model_layer, _ptr(attn_out), _ptr(residual_in), _ptr(next_norm_weight),
            _ptr(layer_out), _ptr(next_norm_out), int(attn_out.shape[0]), _stream(torch)))
        return layer_out, next_norm_out

    def rmsnorm(self, x: Any, weight: Any, residual: Any = None, eps: float = 1.0e-6) -> tuple[Any, Any]:
        torch = self._torch
        rows = int(x.numel() // HIDDEN)
        norm_out = torch.empty_like(x)
        residual_out = torch.empty_like(x) if residual is not None else None
        self.lib.check(self.lib.aima_moe_rmsnorm_launch(
            _ptr(x), _ptr(residual), _ptr(weight), _ptr(residual_out), _ptr(norm_out), rows, eps,
            _stream(torch)))
        return residual_out, norm_out

    def gemv(self, weight: Any, x: Any) -> Any:
        torch = self._torch
        m, k = int(weight.shape[0]), int(weight.shape[1])
        out = torch.empty(m, dtype=torch.bfloat16, device=weight.device)
        self.lib.check(self.lib.aima_moe_gemv_bf16_launch(_ptr(weight), _ptr(x), _ptr(out), m, k, _stream(torch)))
        return out

    # -- expert parallelism ---------------------------------------------------
    def ep_local_buffer(self) -> tuple[int, int]:
        pointer, size = c_void_p(), c_uint64()
        self.lib.check(self.lib.aima_moe_ep_local_buffer(self.handle, ctypes.byref(pointer), ctypes.byref(size)))
        return int(pointer.value), int(size.value)

    def ep_export(self) -> bytes:
        buffer = ctypes.create_string_buffer(64)
        self.lib.check(self.lib.aima_moe_ep_export(self.handle, buffer))
        return buffer.raw

    def ep_connect(self, peer: int, ipc_handle: bytes | None = None, pointer: int | None = None) -> None:
        handle_buffer = ctypes.create_string_buffer(ipc_handle, 64) if ipc_handle is not None else None
        self.lib.check(self.lib.aima_moe_ep_connect(
            self.handle, peer, handle_buffer, c_void_p(pointer) if pointer is not None else None))

    def ep_connect_all(self, group: Any = None) -> None:
        """One process per GPU: all-gathers the 64-byte IPC handles over torch.distributed
        (any backend; the payload is a CPU byte tensor for gloo, a CUDA one for nccl) and maps
        every peer's exchange buffer."""
        handles = exchange_ipc_handles(self.ep_export(), self.config.rank, self.config.world, group)
        for peer, handle in enumerate(handles):
            if peer != self.config.rank:
                self.ep_connect(peer, ipc_handle=handle)

    def set_tracing(self, enabled: bool) -> None:
        self.lib.check(self.lib.aima_moe_set_tracing(self.handle, int(enabled)))

    def debug_set_decode_epoch(self, epoch: int) -> None:
        """Qualification: presets the epoch counter the decode kernel's exchange tags derive from."""
        self.lib.check(self.lib.aima_moe_debug_set_decode_epoch(self.handle, epoch & 0xFFFFFFFF))

    def decode_timeline(self) -> list[list[int]]:
        """Per layer of the last traced decode launch: 12 GPU nanosecond stamps."""
        capacity = MAX_LAYERS * 12
        buffer = (c_uint64 * capacity)()
        written = c_uint32()
        self.lib.check(self.lib.aima_moe_read_decode_timeline(self.handle, buffer, capacity, ctypes.byref(written)))
        values = list(buffer[: written.value])
        return [values[i:i + 12] for i in range(0, len(values), 12)]

    def decode_block_timelines(self) -> list[list[list[int]]]:
        """[block][layer][16] GPU nanosecond stamps of the last traced decode launch."""
        capacity = 256 * MAX_LAYERS * 16
        buffer = (c_uint64 * capacity)()
        blocks, layers = c_uint32(), c_uint32()
        self.lib.check(self.lib.aima_moe_read_decode_block_timelines(self.handle, buffer, capacity,
                                                                     ctypes.byref(blocks), ctypes.byref(layers)))
        n_layers = layers.value
        return [[list(buffer[(b * n_layers + l) * 16:(b * n_layers + l + 1) * 16]) for l in range(n_layers)]
                for b in range(blocks.value)]

    def gemm(self, a: Any, b: Any) -> Any:
        """D[m, n] = A[m, k] . B[n, k]^T on the tensor cores (BF16 in/out)."""
        torch = self._torch
        m, k = int(a.shape[0]), int(a.shape[1])
        n = int(b.shape[0])
        d = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
        self.lib.check(self.lib.aima_moe_gemm_bf16_launch(self.handle, _ptr(a), _ptr(b), _ptr(d), m, n, k,
                                                          _stream(torch)))
        return d

    EP_PREFILL_STAGES = ("route", "routing_exchange", "plan", "dispatch", "experts", "row_return",
                         "shared_wait_combine")

    def ep_prefill_stages(self) -> dict[str, float]:
        """Milliseconds per stage of the last traced expert-parallel prefill call."""
        buffer = (c_float * 7)()
        written = c_uint32()
        self.lib.check(self.lib.aima_moe_read_ep_prefill_stages(self.handle, buffer, 7, ctypes.byref(written)))
        return {name: float(buffer[i]) for i, name in enumerate(self.EP_PREFILL_STAGES[: written.value])}

    def sync_metrics(self) -> Metrics:
        metrics = Metrics()
        metrics.struct_bytes = ctypes.sizeof(Metrics)
        self.lib.check(self.lib.aima_moe_sync_metrics(self.handle, ctypes.byref(metrics)))
        return metrics

    def stats(self) -> dict[str, Any]:
        return {"prepared": self.handle is not None, "call_counts": dict(self.calls),
                "library": str(self.lib.path)}

    def release(self) -> None:
        if getattr(self, "handle", None):
            self.lib.aima_moe_release(self.handle)
            self.handle = None
            self._keepalive.clear()

    def __del__(self) -> None:  # best effort
        try:
            self.release()
        except Exception:
            pass


class LmHead:
    """LM head with a certified top-1 over a raw [rows, 2048] BF16 matrix on the device: the binding of
    aima_moe_lm_head_* (the reference's int8_certified_global_tie variant,
    benchmarks/shape-lab/four_layer_mini_engine.py:8656-8678)."""

    def __init__(self, weight: Any, library: MoeLibrary | None = None) -> None:
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("aima_moe needs a CUDA device (sm_100a); there is no CPU fallback")
        self._torch = torch
        self.lib = library or load_library()
        self.weight = weight                      # kept alive: the exact candidate logits read it
        self.rows = int(weight.shape[0])
        handle = c_void_p()
        self.lib.check(self.lib.aima_moe_lm_head_build(_ptr(weight), self.rows, ctypes.byref(handle), _stream(torch)))
        self.handle = handle

    def views(self) -> tuple[Any, Any, Any]:
        """(q_weight int8 [rows, 2048], scales f32 [rows], residual_l2 f32 [rows]) copied to host tensors."""
        torch = self._torch
        q, s, r = c_void_p(), c_void_p(), c_void_p()
        self.lib.check(self.lib.aima_moe_lm_head_views(self.handle, ctypes.byref(q), ctypes.byref(s), ctypes.byref(r)))
        torch.cuda.synchronize()

        class _DeviceArray:  # zero-copy view of library-owned device memory
            def __init__(self, pointer: int, shape: tuple, typestr: str) -> None:
                self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (pointer, False),
                                                 "version": 2}

        device = self.weight.device
        out_q = torch.as_tensor(_DeviceArray(q.value, (self.rows, HIDDEN), "|i1"), device=device).cpu()
        out_s = torch.as_tensor(_DeviceArray(s.value, (self.rows,), "<f4"), device=device).cpu()
        out_r = torch.as_tensor(_DeviceArray(r.value, (self.rows,), "<f4"), device=device).cpu()
        return out_q, out_s, out_r

    def launch(self, hidden: Any, logits: Any | None = None) -> Any:
        torch = self._torch
        if logits is None:
            logits = torch.empty(self.rows, dtype=torch.float32, device=hidden.device)
        self.lib.check(self.lib.aima_moe_lm_head_launch(self.handle, _ptr(hidden), _ptr(logits), _stream(torch)))
        return logits

    def result(self) -> LmHeadResult:
        result = LmHeadResult()
        self.lib.check(self.lib.aima_moe_lm_head_read_result(self.handle, ctypes.byref(result)))
        return result

    def release(self) -> None:
        if self.handle is not None and self.handle.value:
            self.lib.aima_moe_lm_head_release(self.handle)
            self.handle = c_void_p()


class StripedImage:
    """Binding of aima_moe_image_*: the two-lane striped weight image (layout plan, builder, scatter ingest with
    the device checksum).  `tensors` maps names to contiguous CPU tensors whose byte size is a multiple of 8."""

    def __init__(self, library: MoeLibrary | None = None) -> None:
        self.lib = library or load_library()

    def plan(self, names: list[str], payload_bytes: list[int]) -> dict:
        count = len(names)
        sizes = (c_uint64 * count)(*payload_bytes)
        c_names = (ctypes.c_char_p * count)(*[name.encode() for name in names])
        lane = (c_uint32 * count)()
        lane_offset = (c_uint64 * count)()
        aggregate = (c_uint64 * count)()
        lane_bytes = (c_uint64 * 2)()
        self.lib.check(self.lib.aima_moe_image_plan(sizes, c_names, count, lane, lane_offset, aggregate, lane_bytes))
        return {"lane": list(lane), "lane_offset": list(lane_offset), "aggregate_offset": list(aggregate),
                "lane_bytes": list(lane_bytes)}

    def checksum(self, tensor: Any, start: tuple[int, int] = (0, 0)) -> tuple[int, int]:
        xor_value, sum_value = c_uint64(start[0]), c_uint64(start[1])
        nbytes = tensor.numel() * tensor.element_size()
        self.lib.check(self.lib.aima_moe_image_checksum_host(
            c_void_p(tensor.data_ptr()), nbytes, ctypes.byref(xor_value), ctypes.byref(sum_value)))
        return int(xor_value.value), int(sum_value.value)

    def build(self, lane0_path: str, lane1_path: str, names: list[str], tensors: dict) -> dict:
        sizes = [tensors[name].numel() * tensors[name].element_size() for name in names]
        plan = self.plan(names, sizes)
        count = len(names)
        pointers = (c_void_p * count)(*[tensors[name].data_ptr() for name in names])
        xor_value, sum_value = c_uint64(), c_uint64()
        self.lib.check(self.lib.aima_moe_image_build(
            str(lane0_path).encode(), str(lane1_path).encode(), pointers, (c_uint64 * count)(*sizes),
            (c_uint32 * count)(*plan["lane"]), (c_uint64 * count)(*plan["lane_offset"]), count,
            (c_uint64 * 2)(*plan["lane_bytes"]), ctypes.byref(xor_value), ctypes.byref(sum_value)))
        plan.update({"payload_bytes": sizes, "xor": int(xor_value.value), "sum": int(sum_value.value),
                     "names": list(names)})
        return plan

    def safetensors_index(self, path: str) -> list[dict]:
        """Tensors of one safetensors shard: name, dtype, shape and absolute byte range in the file."""
        count = c_uint64()
        self.lib.check(self.lib.aima_moe_safetensors_index(str(path).encode(), None, 0, ctypes.byref(count)))
        entries = (SafetensorsEntry * max(count.value, 1))()
        self.lib.check(self.lib.aima_moe_safetensors_index(str(path).encode(), entries, count.value, ctypes.byref(count)))
        return [{"name": e.name.decode(), "dtype": e.dtype.decode(), "shape": list(e.shape[:e.rank]),
                 "begin": int(e.data_begin), "end": int(e.data_end)} for e in entries[:count.value]]

    def build_from_files(self, lane0_path: str, lane1_path: str, sources: list[dict]) -> dict:
        """sources: dicts with name, path, begin, end (e.g. from safetensors_index plus the shard's path)."""
        names = [entry["name"] for entry in sources]
        sizes = [entry["end"] - entry["begin"] for entry in sources]
        plan = self.plan(names, sizes)
        count = len(sources)
        xor_value, sum_value = c_uint64(), c_uint64()
        self.lib.check(self.lib.aima_moe_image_build_from_files(
            str(lane0_path).encode(), str(lane1_path).encode(),
            (ctypes.c_char_p * count)(*[str(entry["path"]).encode() for entry in sources]),
            (c_uint64 * count)(*[entry["begin"] for entry in sources]), (c_uint64 * count)(*sizes),
            (c_uint32 * count)(*plan["lane"]), (c_uint64 * count)(*plan["lane_offset"]), count,
            (c_uint64 * 2)(*plan["lane_bytes"]), ctypes.byref(xor_value), ctypes.byref(sum_value)))
        plan.update({"payload_bytes": sizes, "xor": int(xor_value.value), "sum": int(sum_value.value), "names": names})
        return plan

    def scatter_ingest(self, lane0_path: str, lane1_path: str, ranges: list[tuple[int, int]], destinations: list,
                       lane_bytes: list[int], chunk_bytes: int = 8 << 20,
                       expected: tuple[int, int] | None = None) -> ImageIngestResult:
        """ranges: (aggregate offset, bytes) per destination tensor (device, contiguous)."""
        count = len(ranges)
        result = ImageIngestResult()
        self.lib.check(self.lib.aima_moe_image_scatter_ingest(
            str(lane0_path).encode(), str(lane1_path).encode(), (c_uint64 * count)(*[r[0] for r in ranges]),
            (c_uint64 * count)(*[r[1] for r in ranges]), (c_uint64 * count)(*[t.data_ptr() for t in destinations]),
            count, lane_bytes[0], lane_bytes[1], chunk_bytes, 0 if expected is None else 1,
            0 if expected is None else expected[0], 0 if expected is None else expected[1], ctypes.byref(result)))
        return result
