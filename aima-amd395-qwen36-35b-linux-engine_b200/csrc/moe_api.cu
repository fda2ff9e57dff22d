// Host side of the C ABI declared in include/aima_moe.h.
//
// Mirrors the fail-closed style of the reference runtime's owners
// (native/src/native_moe_prefill.hip.cpp:44-87, 550-599, 711-715): every size,
// residency and alias rule is checked before anything is enqueued, each check
// has its own message, and nothing throws across the boundary.
#include "../../include/aima_moe.h"

#include "decode_kernel.cuh"
#include "pointwise.cuh"
#include "grouped_gemm.cuh"
#include "prefill.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

using namespace aima;

namespace {

thread_local char g_last_error[512] = "";

int fail(int code, const char* format, ...) {
  va_list args;
  va_start(args, format);
  std::vsnprintf(g_last_error, sizeof g_last_error, format, args);
  va_end(args);
  return code;
}

int fail_cuda(cudaError_t error, const char* operation) {
  std::snprintf(g_last_error, sizeof g_last_error, "%s: %s (%s)", operation,
                cudaGetErrorName(error), cudaGetErrorString(error));
  (void)cudaGetLastError();
  return static_cast<int>(error);
}

constexpr uint64_t kRouterBytes = 2ull * kExperts * kHidden;
constexpr uint64_t kGateUpBytesPerExpert = 2ull * 2 * kInter * kHidden;
constexpr uint64_t kDownBytesPerExpert = 2ull * kHidden * kInter;
constexpr uint64_t kSharedGateBytes = 2ull * kHidden;
constexpr uint64_t kSharedProjBytes = 2ull * kSharedInter * kHidden;
constexpr uint64_t kNormBytes = 2ull * kHidden;

size_t align_up(size_t value, size_t alignment) {
  return (value + alignment - 1) / alignment * alignment;
}

}  // namespace

namespace aima {
// Lets other translation units of the library report through aima_moe_last_error_string().
void set_last_error_message(const char* message) {
  std::snprintf(g_last_error, sizeof g_last_error, "%s", message);
}
}  // namespace aima

struct aima_moe_handle {
  aima_moe_config config{};
  int device = -1;
  int sm_count = 0;
  int decode_grid = 0;
  int experts_local = 0;
  int expert_lo = 0;
  LayerPtrs host_layers[kMaxLayers]{};
  bool bound[kMaxLayers]{};
  LayerPtrs* dev_layers = nullptr;

  // decode scratch (one allocation)
  uint8_t* decode_scratch = nullptr;
  size_t decode_scratch_bytes = 0;
  // [exchange area, cleared together: sync words | status | logits | xbuf0 | xbuf1] act | gate
  uint32_t* xbuf0 = nullptr;
  uint32_t* xbuf1 = nullptr;
  unsigned long long* logits = nullptr;
  uint32_t* act = nullptr;
  unsigned* epoch_base = nullptr;
  int* status = nullptr;

  PrefillWorkspace prefill;

  // expert parallelism (world > 1): this GPU's exchange buffer and the peers' mapped buffers
  // layout of one exchange allocation: [decode slot products kEpExchangeBytes][prefill region]
  unsigned long long* ep_local = nullptr;
  size_t ep_bytes = 0;
  EpPrefill ep_prefill;
  unsigned long long* ep_peers[8] = {};
  void* ep_ipc_opened[8] = {};
  float* router_row_norms = nullptr;        // [kMaxLayers][256], device, filled by bind_layer
  unsigned long long* timeline = nullptr;   // [kDecodeMaxBlocks][kMaxLayers][kDecodeTraceSlots], device
  bool tracing = false;
  uint32_t traced_layers = 0;

  const float* router_bias = nullptr;
  int quant_eighths = 0;
  // qualification: routing supplied by the harness for single-layer prefill calls of exactly this many tokens
  const int32_t* forced_ids = nullptr;
  const void* forced_weights = nullptr;
  uint32_t forced_tokens = 0;

  aima_moe_metrics metrics{};
  cudaStream_t last_stream = nullptr;
  std::mutex mutex;
};

namespace {

int validate_config(const aima_moe_config* config) {
  if (config == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "config is null");
  if (config->struct_bytes != sizeof(aima_moe_config))
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "aima_moe_config size mismatch: got %u, built for %zu",
                config->struct_bytes, sizeof(aima_moe_config));
  if (config->hidden != kHidden || config->experts != kExperts || config->top_k != kTopK ||
      config->expert_inter != kInter || config->shared_inter != kSharedInter)
    return fail(AIMA_MOE_ERR_UNSUPPORTED,
                "only hidden 2048 / 256 experts / top-8 / intermediate 512 / shared 512 is built");
  if (config->layers == 0 || config->layers > kMaxLayers)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "layers must be 1..%d", kMaxLayers);
  if (config->world != 1 && config->world != 2 && config->world != 4 && config->world != 8)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "world must be 1, 2, 4 or 8");
  if (config->rank >= config->world)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "rank %u out of range for world %u",
                config->rank, config->world);
  if (!(config->rms_eps > 0.0f) || !(config->rms_eps < 1.0f))
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "rms_eps must be in (0, 1)");
  if (config->max_prefill_tokens > 262144u)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "max_prefill_tokens exceeds 262144");
  return AIMA_MOE_OK;
}

// exchange area: sync words 256 B, status 256 B, replicated tagged logits and two replicated tagged vectors
constexpr size_t kLogitsBytes = static_cast<size_t>(kDecodeLogitWords) * 8;   // real + predicted
constexpr size_t kXbufBytes = static_cast<size_t>(kDecodeReplicas) * kHidden * 4;
constexpr size_t kExchangeBytes = 256 + 256 + kLogitsBytes + 2 * kXbufBytes;

size_t decode_scratch_size() {
  return kExchangeBytes + align_up(static_cast<size_t>(kDecodeReplicas) * kDecodeActStride * 4, 256);
}

// AIMA_MOE_DECODE_IN_FLIGHT in the environment overrides how many ring items a block of the decode
// kernel may have outstanding (0: no limit).
int decode_max_in_flight() {
  static const int value = [] {
    const char* v = std::getenv("AIMA_MOE_DECODE_IN_FLIGHT");
    return (v != nullptr && v[0] != '\0') ? std::atoi(v) : kDecodeDefaultInFlight;
  }();
  return value;
}

int check_device_tensor(const void* pointer, uint64_t bytes, uint64_t expected,
                        const char* name) {
  if (pointer == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "weight %s is null", name);
  if (bytes != expected)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "weight %s has %llu bytes, expected %llu", name,
                static_cast<unsigned long long>(bytes), static_cast<unsigned long long>(expected));
  if (reinterpret_cast<uintptr_t>(pointer) % 16 != 0)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "weight %s is not 16-byte aligned", name);
  cudaPointerAttributes attributes{};
  const cudaError_t error = cudaPointerGetAttributes(&attributes, pointer);
  if (error != cudaSuccess) return fail_cuda(error, "cudaPointerGetAttributes");
  if (attributes.type != cudaMemoryTypeDevice && attributes.type != cudaMemoryTypeManaged)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "weight %s is not device resident", name);
  return AIMA_MOE_OK;
}

bool ranges_overlap(const void* a, size_t a_bytes, const void* b, size_t b_bytes) {
  const uintptr_t a0 = reinterpret_cast<uintptr_t>(a);
  const uintptr_t b0 = reinterpret_cast<uintptr_t>(b);
  return a0 < b0 + b_bytes && b0 < a0 + a_bytes;
}

// A handle's buffers, layer table and kernels' attributes belong to the device it was prepared on.
int check_current_device(const aima_moe_handle* handle) {
  int device = -1;
  const cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return fail_cuda(error, "cudaGetDevice");
  if (device != handle->device)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT,
                "the handle was prepared on device %d but device %d is current; make its device current first",
                handle->device, device);
  return AIMA_MOE_OK;
}

int reset_decode_sync(aima_moe_handle* handle) {
  // tags restart from zero, so every tagged word must be cleared with the counters
  cudaError_t error = cudaMemset(handle->decode_scratch, 0, kExchangeBytes);
  if (error == cudaSuccess && handle->ep_local != nullptr) {
    error = cudaMemset(handle->ep_local, 0, handle->ep_bytes);
    handle->ep_prefill.epoch = 0;
  }
  if (error != cudaSuccess) return fail_cuda(error, "cudaMemset decode exchange area");
  return AIMA_MOE_OK;
}

int launch_decode_range(aima_moe_handle* handle, uint32_t first_layer, uint32_t n_layers,
                        const void* x_in, void* x_out, const aima_moe_debug_views* debug,
                        void* stream) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if (const int wrong_device = check_current_device(handle); wrong_device != AIMA_MOE_OK) return wrong_device;
  if (x_in == nullptr || x_out == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "decode input/output is null");
  if (n_layers == 0 || first_layer >= handle->config.layers ||
      n_layers > handle->config.layers - first_layer)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "decode layer range [%u, %u) is out of range",
                first_layer, first_layer + n_layers);
  for (uint32_t layer = first_layer; layer < first_layer + n_layers; ++layer) {
    if (!handle->bound[layer])
      return fail(AIMA_MOE_ERR_NOT_BOUND, "layer %u has no bound weights", layer);
    if (handle->host_layers[layer].norm_weight == nullptr)
      return fail(AIMA_MOE_ERR_NOT_BOUND, "layer %u has no post-attention norm weight", layer);
  }
  if (ranges_overlap(x_in, kHidden * 2, x_out, kHidden * 2))
    return fail(AIMA_MOE_ERR_ALIAS, "decode output aliases its input");
  if (reinterpret_cast<uintptr_t>(x_in) % 16 != 0 || reinterpret_cast<uintptr_t>(x_out) % 16 != 0)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "decode vectors must be 16-byte aligned");
  if (debug != nullptr && debug->struct_bytes != sizeof(aima_moe_debug_views))
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "aima_moe_debug_views size mismatch");
  for (uint32_t peer = 0; peer < handle->config.world; ++peer) {
    if (handle->config.world > 1 && handle->ep_peers[peer] == nullptr)
      return fail(AIMA_MOE_ERR_NOT_BOUND, "expert-parallel peer %u is not connected (aima_moe_ep_connect)", peer);
  }

  DecodeParams params{};
  params.layers = handle->dev_layers;
  params.x_in = static_cast<const __nv_bfloat16*>(x_in);
  params.x_out = static_cast<__nv_bfloat16*>(x_out);
  params.xbuf0 = handle->xbuf0;
  params.xbuf1 = handle->xbuf1;
  params.logits = handle->logits;
  params.act = handle->act;
  params.epoch_base = handle->epoch_base;
  params.status = handle->status;
  params.router_bias = handle->router_bias;
  params.quant_eighths = handle->quant_eighths;
  params.speculate = (handle->config.flags & AIMA_MOE_FLAG_NO_DECODE_PREDICTION) == 0 ? 1 : 0;
  params.max_in_flight = decode_max_in_flight();
  params.eps = handle->config.rms_eps;
  params.first_layer = static_cast<int>(first_layer);
  params.n_layers = static_cast<int>(n_layers);
  params.expert_lo = handle->expert_lo;
  params.expert_hi = handle->expert_lo + handle->experts_local;
  for (int peer = 0; peer < 8; ++peer) params.ep_dots[peer] = handle->ep_peers[peer];
  params.world = static_cast<int>(handle->config.world);
  params.rank = static_cast<int>(handle->config.rank);
  params.timeline = handle->tracing ? handle->timeline : nullptr;
  if (handle->tracing) handle->traced_layers = n_layers;
  if (debug != nullptr) {
    params.dbg_h2 = static_cast<__nv_bfloat16*>(debug->h2);
    params.dbg_logits = static_cast<float*>(debug->router_logits);
    params.dbg_ids = static_cast<int*>(debug->topk_ids);
    params.dbg_scores = static_cast<float*>(debug->topk_scores);
    params.dbg_weights = static_cast<__nv_bfloat16*>(debug->topk_weights);
    params.dbg_shared_scaled = static_cast<__nv_bfloat16*>(debug->shared_scaled);
    params.dbg_routed = static_cast<__nv_bfloat16*>(debug->routed);
    params.dbg_slot_dots = static_cast<float*>(debug->slot_dots);
  }
  const cudaError_t error =
      launch_moe_decode(params, handle->decode_grid, static_cast<cudaStream_t>(stream));
  if (error != cudaSuccess) return fail_cuda(error, "launch moe_decode_persistent_kernel");
  handle->last_stream = static_cast<cudaStream_t>(stream);
  handle->metrics.decode_calls += 1;
  handle->metrics.kernel_launches += 1;
  return AIMA_MOE_OK;
}

}  // namespace

extern "C" {

#define AIMA_EXPORT __attribute__((visibility("default")))

AIMA_EXPORT uint32_t aima_moe_abi_version(void) { return (1u << 16) | 0u; }

AIMA_EXPORT const char* aima_moe_last_error_string(void) { return g_last_error; }

AIMA_EXPORT int aima_moe_query_workspace(const aima_moe_config* config, uint64_t* bytes) {
  const int status = validate_config(config);
  if (status != AIMA_MOE_OK) return status;
  if (bytes == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "bytes is null");
  *bytes = decode_scratch_size() + sizeof(LayerPtrs) * kMaxLayers +
           prefill_workspace_bytes(config->max_prefill_tokens);
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_prepare(const aima_moe_config* config, aima_moe_handle** out_handle) {
  int status = validate_config(config);
  if (status != AIMA_MOE_OK) return status;
  if (out_handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle out-pointer is null");
  *out_handle = nullptr;

  int device = -1;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(AIMA_MOE_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(error));
  }
  cudaDeviceProp properties{};
  error = cudaGetDeviceProperties(&properties, device);
  if (error != cudaSuccess) return fail_cuda(error, "cudaGetDeviceProperties");
  if (properties.major != 10)
    return fail(AIMA_MOE_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                device, properties.major, properties.minor);
  const int grid = properties.multiProcessorCount < kDecodeMaxBlocks
                       ? properties.multiProcessorCount
                       : kDecodeMaxBlocks;
  if (grid < kDecodeMinBlocks)
    return fail(AIMA_MOE_ERR_UNSUPPORTED, "device exposes %d SMs; the decode kernel needs at least %d",
                properties.multiProcessorCount, kDecodeMinBlocks);
  if (!properties.cooperativeLaunch)
    return fail(AIMA_MOE_ERR_UNSUPPORTED, "device does not support cooperative launch");

  aima_moe_handle* handle = new (std::nothrow) aima_moe_handle();
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INTERNAL, "out of host memory");
  handle->config = *config;
  handle->device = device;
  handle->sm_count = properties.multiProcessorCount;
  handle->decode_grid = grid;
  handle->experts_local = kExperts / static_cast<int>(config->world);
  handle->expert_lo = handle->experts_local * static_cast<int>(config->rank);

  auto cleanup = [&](int code) {
    if (handle->timeline) cudaFree(handle->timeline);
    if (handle->ep_local) cudaFree(handle->ep_local);
    if (handle->router_row_norms) cudaFree(handle->router_row_norms);
    if (handle->dev_layers) cudaFree(handle->dev_layers);
    if (handle->decode_scratch) cudaFree(handle->decode_scratch);
    prefill_workspace_free(&handle->prefill);
    delete handle;
    return code;
  };

  error = cudaMalloc(&handle->dev_layers, sizeof(LayerPtrs) * kMaxLayers);
  if (error != cudaSuccess) return cleanup(fail_cuda(error, "cudaMalloc layer table"));
  error = cudaMemset(handle->dev_layers, 0, sizeof(LayerPtrs) * kMaxLayers);
  if (error != cudaSuccess) return cleanup(fail_cuda(error, "cudaMemset layer table"));

  error = cudaMalloc(&handle->timeline, sizeof(unsigned long long) * kDecodeMaxBlocks * kMaxLayers * kDecodeTraceSlots);
  if (error != cudaSuccess) return cleanup(fail_cuda(error, "cudaMalloc decode timeline"));
  if (config->world > 1) {
    handle->ep_prefill.world = static_cast<int>(config->world);
    handle->ep_prefill.rank = static_cast<int>(config->rank);
    handle->ep_bytes = kEpExchangeBytes;
    if (config->max_prefill_tokens > 0) {
      handle->ep_bytes += ep_prefill_region_bytes(static_cast<int>(config->max_prefill_tokens),
                                                  static_cast<int>(config->world), &handle->ep_prefill.layout);
    }
    error = cudaMalloc(&handle->ep_local, handle->ep_bytes);
    if (error == cudaSuccess) error = cudaMemset(handle->ep_local, 0, handle->ep_bytes);
    if (error != cudaSuccess) return cleanup(fail_cuda(error, "cudaMalloc expert-parallel exchange buffer"));
    handle->ep_peers[config->rank] = handle->ep_local;
  }
  error = cudaMalloc(&handle->router_row_norms, sizeof(float) * kMaxLayers * kExperts);
  if (error != cudaSuccess) return cleanup(fail_cuda(error, "cudaMalloc router row norms"));
  handle->decode_scratch_bytes = decode_scratch_size();
  error = cudaMalloc(&handle->decode_scratch, handle->decode_scratch_bytes);
  if (error != cudaSuccess) return cleanup(fail_cuda(error, "cudaMalloc decode scratch"));
  error = cudaMemset(handle->decode_scratch, 0, handle->decode_scratch_bytes);
  if (error != cudaSuccess) return cleanup(fail_cuda(error, "cudaMemset decode scratch"));
  uint8_t* cursor = handle->decode_scratch;
  handle->epoch_base = reinterpret_cast<unsigned*>(cursor + 192);
  cursor += 256;
  handle->status = reinterpret_cast<int*>(cursor); cursor += 256;
  handle->logits = reinterpret_cast<unsigned long long*>(cursor); cursor += kLogitsBytes;
  handle->xbuf0 = reinterpret_cast<uint32_t*>(cursor); cursor += kXbufBytes;
  handle->xbuf1 = reinterpret_cast<uint32_t*>(cursor); cursor += kXbufBytes;
  handle->act = reinterpret_cast<uint32_t*>(cursor);

  if (config->max_prefill_tokens > 0) {
    status = prefill_workspace_allocate(&handle->prefill, config->max_prefill_tokens,
                                        handle->sm_count, g_last_error, sizeof g_last_error);
    if (status != AIMA_MOE_OK) return cleanup(status);
    handle->prefill.status = handle->status;
    handle->prefill.use_simt_gemm = (config->flags & AIMA_MOE_FLAG_SIMT_PRODUCTS) != 0;
    handle->prefill.exact_router = (config->flags & AIMA_MOE_FLAG_EXACT_ROUTER) != 0;
    handle->prefill.router_audit_stride = (config->flags & AIMA_MOE_FLAG_AUDIT_ROUTER) != 0 ? 64 : 0;
    handle->prefill.fused_dispatch = (config->flags & AIMA_MOE_FLAG_MATERIALIZED_DISPATCH) == 0;
    handle->prefill.pair_products = (config->flags & AIMA_MOE_FLAG_TWO_SM_PRODUCTS) != 0 && config->world == 1;
    handle->prefill.ep_parts = (config->flags & AIMA_MOE_FLAG_EP_PIPELINE_4)   ? 4
                               : (config->flags & AIMA_MOE_FLAG_EP_PIPELINE_2) ? 2
                                                                               : 1;
    // A/B switch: AIMA_MOE_EP_COPY_RETURN in the environment keeps the copy kernel that returns the rows
    handle->prefill.ep_fused_return = std::getenv("AIMA_MOE_EP_COPY_RETURN") == nullptr;
    handle->prefill.ep_fused_dispatch = std::getenv("AIMA_MOE_EP_COPY_DISPATCH") == nullptr;
  }
  handle->metrics.struct_bytes = sizeof(aima_moe_metrics);
  handle->metrics.workspace_bytes = handle->decode_scratch_bytes + sizeof(LayerPtrs) * kMaxLayers +
                                    handle->prefill.total_bytes;
  *out_handle = handle;
  g_last_error[0] = '\0';
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_bind_layer(aima_moe_handle* handle, uint32_t layer,
                                    const aima_moe_layer_weights* weights) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if (const int wrong_device = check_current_device(handle); wrong_device != AIMA_MOE_OK) return wrong_device;
  if (weights == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "weights is null");
  if (weights->struct_bytes != sizeof(aima_moe_layer_weights))
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "aima_moe_layer_weights size mismatch");
  if (layer >= handle->config.layers)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "layer %u out of range (layers = %u)", layer,
                handle->config.layers);
  const uint64_t local = static_cast<uint64_t>(handle->experts_local);
  int status;
  if ((status = check_device_tensor(weights->router, weights->router_bytes, kRouterBytes,
                                    "mlp.gate.weight")) != AIMA_MOE_OK) return status;
  if ((status = check_device_tensor(weights->expert_gate_up, weights->expert_gate_up_bytes,
                                    local * kGateUpBytesPerExpert,
                                    "mlp.experts.gate_up_proj")) != AIMA_MOE_OK) return status;
  if ((status = check_device_tensor(weights->expert_down, weights->expert_down_bytes,
                                    local * kDownBytesPerExpert,
                                    "mlp.experts.down_proj")) != AIMA_MOE_OK) return status;
  if ((status = check_device_tensor(weights->shared_expert_gate, weights->shared_expert_gate_bytes,
                                    kSharedGateBytes, "mlp.shared_expert_gate.weight")) != AIMA_MOE_OK)
    return status;
  if ((status = check_device_tensor(weights->shared_gate_proj, weights->shared_gate_proj_bytes,
                                    kSharedProjBytes, "mlp.shared_expert.gate_proj.weight")) != AIMA_MOE_OK)
    return status;
  if ((status = check_device_tensor(weights->shared_up_proj, weights->shared_up_proj_bytes,
                                    kSharedProjBytes, "mlp.shared_expert.up_proj.weight")) != AIMA_MOE_OK)
    return status;
  if ((status = check_device_tensor(weights->shared_down_proj, weights->shared_down_proj_bytes,
                                    kSharedProjBytes, "mlp.shared_expert.down_proj.weight")) != AIMA_MOE_OK)
    return status;
  if (weights->post_attention_norm != nullptr &&
      (status = check_device_tensor(weights->post_attention_norm, weights->post_attention_norm_bytes,
                                    kNormBytes, "post_attention_layernorm.weight")) != AIMA_MOE_OK)
    return status;

  LayerPtrs pointers{};
  pointers.router = static_cast<const __nv_bfloat16*>(weights->router);
  pointers.expert_gate_up = static_cast<const __nv_bfloat16*>(weights->expert_gate_up);
  pointers.expert_down = static_cast<const __nv_bfloat16*>(weights->expert_down);
  pointers.shared_gate = static_cast<const __nv_bfloat16*>(weights->shared_expert_gate);
  pointers.shared_gate_proj = static_cast<const __nv_bfloat16*>(weights->shared_gate_proj);
  pointers.shared_up_proj = static_cast<const __nv_bfloat16*>(weights->shared_up_proj);
  pointers.shared_down_proj = static_cast<const __nv_bfloat16*>(weights->shared_down_proj);
  pointers.norm_weight = static_cast<const __nv_bfloat16*>(weights->post_attention_norm);
  cudaError_t error = cudaMemcpy(handle->dev_layers + layer, &pointers, sizeof pointers,
                                 cudaMemcpyHostToDevice);
  if (error != cudaSuccess) return fail_cuda(error, "cudaMemcpy layer table entry");
  error = launch_router_row_norms(pointers.router, handle->router_row_norms + layer * kExperts, nullptr);
  if (error == cudaSuccess) error = cudaStreamSynchronize(nullptr);
  if (error != cudaSuccess) return fail_cuda(error, "router row norms");
  handle->host_layers[layer] = pointers;
  handle->bound[layer] = true;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_set_router_hooks(aima_moe_handle* handle, const void* bias_f32,
                                          int quantize_eighths) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  handle->router_bias = static_cast<const float*>(bias_f32);
  handle->quant_eighths = quantize_eighths ? 1 : 0;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_set_forced_routing(aima_moe_handle* handle, const int32_t* ids,
                                            const void* weights_bf16, uint32_t tokens) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if ((ids == nullptr) != (weights_bf16 == nullptr))
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "forced routing needs both ids and weights, or neither");
  if (ids != nullptr && (tokens == 0 || tokens > handle->config.max_prefill_tokens))
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "forced routing for %u tokens does not fit the workspace", tokens);
  if (ids != nullptr && handle->config.world > 1)
    return fail(AIMA_MOE_ERR_UNSUPPORTED, "forced routing is a single-GPU qualification hook");
  handle->forced_ids = ids;
  handle->forced_weights = weights_bf16;
  handle->forced_tokens = ids != nullptr ? tokens : 0;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_decode_launch(aima_moe_handle* handle, uint32_t layer,
                                       const void* after_attn, void* out,
                                       const aima_moe_debug_views* debug, void* stream) {
  return launch_decode_range(handle, layer, 1, after_attn, out, debug, stream);
}

AIMA_EXPORT int aima_moe_decode_stack_launch(aima_moe_handle* handle, uint32_t first_layer,
                                             uint32_t n_layers, const void* x_in, void* x_out,
                                             void* stream) {
  return launch_decode_range(handle, first_layer, n_layers, x_in, x_out, nullptr, stream);
}

AIMA_EXPORT int aima_moe_prefill_launch(aima_moe_handle* handle, uint32_t layer, const void* h2,
                                        const void* residual, void* out, uint32_t tokens,
                                        const aima_moe_debug_views* debug, void* stream) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if (const int wrong_device = check_current_device(handle); wrong_device != AIMA_MOE_OK) return wrong_device;
  if (h2 == nullptr || residual == nullptr || out == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "prefill input/output is null");
  if (tokens == 0) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "tokens is zero");
  if (tokens > handle->config.max_prefill_tokens)
    return fail(AIMA_MOE_ERR_CAPACITY, "tokens %u exceed prepared capacity %u", tokens,
                handle->config.max_prefill_tokens);
  if (layer >= handle->config.layers || !handle->bound[layer])
    return fail(AIMA_MOE_ERR_NOT_BOUND, "layer %u has no bound weights", layer);
  const size_t bytes = static_cast<size_t>(tokens) * kHidden * 2;
  if (ranges_overlap(out, bytes, h2, bytes) || ranges_overlap(out, bytes, residual, bytes))
    return fail(AIMA_MOE_ERR_ALIAS, "prefill output aliases an input");
  if (debug != nullptr && debug->struct_bytes != sizeof(aima_moe_debug_views))
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "aima_moe_debug_views size mismatch");
  if (handle->config.world > 1) {
    if (static_cast<uint64_t>(tokens) * handle->config.world > handle->config.max_prefill_tokens)
      return fail(AIMA_MOE_ERR_CAPACITY, "tokens %u x world %u exceed the prepared global capacity %u", tokens,
                  handle->config.world, handle->config.max_prefill_tokens);
    for (uint32_t peer = 0; peer < handle->config.world; ++peer) {
      if (handle->ep_peers[peer] == nullptr)
        return fail(AIMA_MOE_ERR_NOT_BOUND, "expert-parallel peer %u is not connected (aima_moe_ep_connect)", peer);
      handle->ep_prefill.peers[peer] = reinterpret_cast<uint8_t*>(handle->ep_peers[peer]) + kEpExchangeBytes;
    }
  }
  PrefillCall call{};
  call.layer = handle->host_layers[layer];
  call.h2 = h2;
  call.residual = residual;
  call.out = out;
  call.tokens = static_cast<int>(tokens);
  call.experts_local = handle->experts_local;
  call.router_row_norms = handle->router_row_norms + layer * kExperts;
  call.router_bias = handle->router_bias;
  call.quant_eighths = handle->quant_eighths;
  call.debug = debug;
  if (handle->forced_ids != nullptr) {
    if (handle->forced_tokens != tokens)
      return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "forced routing was set for %u tokens, the call has %u",
                  handle->forced_tokens, tokens);
    call.forced_ids = handle->forced_ids;
    call.forced_weights = handle->forced_weights;
  }
  int launches = 0;
  const int status =
      handle->config.world > 1
          ? prefill_layer_launch_ep(&handle->prefill, call, &handle->ep_prefill, static_cast<cudaStream_t>(stream),
                                    &launches, g_last_error, sizeof g_last_error)
          : prefill_layer_launch(&handle->prefill, call, static_cast<cudaStream_t>(stream), &launches,
                                 g_last_error, sizeof g_last_error);
  if (status != AIMA_MOE_OK) return status;
  handle->last_stream = static_cast<cudaStream_t>(stream);
  handle->metrics.prefill_calls += 1;
  handle->metrics.kernel_launches += static_cast<uint64_t>(launches);
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_prefill_stack_launch(aima_moe_handle* handle, uint32_t first_layer,
                                              uint32_t n_layers, const void* x_in, void* x_out,
                                              uint32_t tokens, void* stream) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if (const int wrong_device = check_current_device(handle); wrong_device != AIMA_MOE_OK) return wrong_device;
  if (x_in == nullptr || x_out == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "prefill stack input/output is null");
  if (tokens == 0 || tokens > handle->config.max_prefill_tokens)
    return fail(AIMA_MOE_ERR_CAPACITY, "tokens %u outside prepared capacity %u", tokens,
                handle->config.max_prefill_tokens);
  if (n_layers == 0 || first_layer >= handle->config.layers ||
      n_layers > handle->config.layers - first_layer)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "prefill layer range is out of range");
  for (uint32_t layer = first_layer; layer < first_layer + n_layers; ++layer) {
    if (!handle->bound[layer] || handle->host_layers[layer].norm_weight == nullptr)
      return fail(AIMA_MOE_ERR_NOT_BOUND, "layer %u lacks weights or its norm weight", layer);
  }
  if (handle->config.world > 1) {
    if (static_cast<uint64_t>(tokens) * handle->config.world > handle->config.max_prefill_tokens)
      return fail(AIMA_MOE_ERR_CAPACITY, "tokens x world exceed the prepared global capacity");
    for (uint32_t peer = 0; peer < handle->config.world; ++peer) {
      if (handle->ep_peers[peer] == nullptr)
        return fail(AIMA_MOE_ERR_NOT_BOUND, "expert-parallel peer %u is not connected", peer);
      handle->ep_prefill.peers[peer] = reinterpret_cast<uint8_t*>(handle->ep_peers[peer]) + kEpExchangeBytes;
    }
  }
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  const size_t bytes = static_cast<size_t>(tokens) * kHidden * 2;
  // x ping-pongs between two workspace buffers; h2 lives in a third.
  const void* current = x_in;
  for (uint32_t step = 0; step < n_layers; ++step) {
    const uint32_t layer = first_layer + step;
    void* target = (step + 1 == n_layers) ? x_out
                   : (step & 1u) ? handle->prefill.stack_x1 : handle->prefill.stack_x0;
    if (target == x_out && ranges_overlap(x_out, bytes, current, bytes)) {
      // final layer would write over its own residual input: stage through a buffer
      target = (step & 1u) ? handle->prefill.stack_x1 : handle->prefill.stack_x0;
    }
    // the first layer's h2 comes from the norm kernel; every later layer's h2 was written by the
    // previous layer's combine kernel (fused exit norm)
    cudaError_t error = cudaSuccess;
    if (step == 0) {
      error = launch_rmsnorm_rows(current, nullptr, handle->host_layers[layer].norm_weight, nullptr,
                                  handle->prefill.stack_h2, static_cast<int>(tokens), handle->config.rms_eps,
                                  cuda_stream);
      if (error != cudaSuccess) return fail_cuda(error, "launch rmsnorm_rows_kernel");
      handle->metrics.kernel_launches += 1;
    }
    PrefillCall call{};
    call.layer = handle->host_layers[layer];
    call.h2 = handle->prefill.stack_h2;
    call.residual = current;
    call.out = target;
    call.tokens = static_cast<int>(tokens);
    call.experts_local = handle->experts_local;
    call.router_row_norms = handle->router_row_norms + layer * kExperts;
    call.router_bias = handle->router_bias;
    call.quant_eighths = handle->quant_eighths;
    call.eps = handle->config.rms_eps;
    if (step + 1 < n_layers) {
      call.next_norm_weight = handle->host_layers[layer + 1].norm_weight;
      call.next_norm_out = handle->prefill.stack_h2;
    }
    int launches = 0;
    const int status =
        handle->config.world > 1
            ? prefill_layer_launch_ep(&handle->prefill, call, &handle->ep_prefill, cuda_stream, &launches,
                                      g_last_error, sizeof g_last_error)
            : prefill_layer_launch(&handle->prefill, call, cuda_stream, &launches, g_last_error,
                                   sizeof g_last_error);
    if (status != AIMA_MOE_OK) return status;
    handle->metrics.kernel_launches += static_cast<uint64_t>(launches);
    if (step + 1 == n_layers && target != x_out) {
      error = cudaMemcpyAsync(x_out, target, bytes, cudaMemcpyDeviceToDevice, cuda_stream);
      if (error != cudaSuccess) return fail_cuda(error, "cudaMemcpyAsync prefill stack output");
    }
    current = target;
  }
  handle->last_stream = cuda_stream;
  handle->metrics.prefill_calls += n_layers;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_prefill_fused_launch(aima_moe_handle* handle, uint32_t layer, const void* attn_out,
                                              const void* residual_in, const void* next_norm_weight,
                                              void* layer_out, void* next_norm_out, uint32_t tokens,
                                              void* stream) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if (const int wrong_device = check_current_device(handle); wrong_device != AIMA_MOE_OK) return wrong_device;
  if (attn_out == nullptr || residual_in == nullptr || layer_out == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "fused prefill input/output is null");
  if ((next_norm_weight == nullptr) != (next_norm_out == nullptr))
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "next_norm_weight and next_norm_out go together");
  if (tokens == 0 || tokens > handle->config.max_prefill_tokens)
    return fail(AIMA_MOE_ERR_CAPACITY, "tokens %u outside prepared capacity %u", tokens,
                handle->config.max_prefill_tokens);
  if (layer >= handle->config.layers || !handle->bound[layer] ||
      handle->host_layers[layer].norm_weight == nullptr)
    return fail(AIMA_MOE_ERR_NOT_BOUND, "layer %u lacks weights or its post-attention norm weight", layer);
  if (handle->config.world > 1)
    return fail(AIMA_MOE_ERR_UNSUPPORTED, "the fused boundary is built for world = 1");
  const size_t bytes = static_cast<size_t>(tokens) * kHidden * 2;
  if (next_norm_out != nullptr && ranges_overlap(next_norm_out, bytes, layer_out, bytes))
    return fail(AIMA_MOE_ERR_ALIAS, "next_norm_out aliases layer_out");
  for (const void* pointer : {attn_out, residual_in, static_cast<const void*>(layer_out),
                              static_cast<const void*>(next_norm_out), next_norm_weight}) {
    if (reinterpret_cast<uintptr_t>(pointer) % 16 != 0)
      return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "fused prefill pointers must be 16-byte aligned");
  }
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  // entry: after_attn = bf16(attn_out + residual_in) and h2 = RMSNorm(after_attn) into the workspace
  cudaError_t error = launch_rmsnorm_rows(attn_out, residual_in, handle->host_layers[layer].norm_weight,
                                          handle->prefill.stack_x0, handle->prefill.stack_h2,
                                          static_cast<int>(tokens), handle->config.rms_eps, cuda_stream);
  if (error != cudaSuccess) return fail_cuda(error, "launch rmsnorm_rows_kernel");
  PrefillCall call{};
  call.layer = handle->host_layers[layer];
  call.h2 = handle->prefill.stack_h2;
  call.residual = handle->prefill.stack_x0;
  call.out = layer_out;
  call.tokens = static_cast<int>(tokens);
  call.experts_local = handle->experts_local;
  call.router_row_norms = handle->router_row_norms + layer * kExperts;
  call.router_bias = handle->router_bias;
  call.quant_eighths = handle->quant_eighths;
  call.eps = handle->config.rms_eps;
  call.next_norm_weight = next_norm_weight;
  call.next_norm_out = next_norm_out;
  int launches = 0;
  const int status = prefill_layer_launch(&handle->prefill, call, cuda_stream, &launches, g_last_error,
                                          sizeof g_last_error);
  if (status != AIMA_MOE_OK) return status;
  handle->last_stream = cuda_stream;
  handle->metrics.prefill_calls += 1;
  handle->metrics.kernel_launches += static_cast<uint64_t>(launches) + 1;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_rmsnorm_launch(const void* x, const void* residual, const void* weight,
                                        void* residual_out, void* norm_out, uint32_t rows,
                                        float eps, void* stream) {
  if (x == nullptr || weight == nullptr || norm_out == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "rmsnorm pointer is null");
  if (rows == 0) return AIMA_MOE_OK;
  const cudaError_t error = launch_rmsnorm_rows(x, residual, weight, residual_out, norm_out,
                                                static_cast<int>(rows), eps,
                                                static_cast<cudaStream_t>(stream));
  if (error != cudaSuccess) return fail_cuda(error, "launch rmsnorm_rows_kernel");
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_gemv_bf16_launch(const void* weight, const void* x, void* out, uint32_t m,
                                          uint32_t k, void* stream) {
  if (weight == nullptr || x == nullptr || out == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "gemv pointer is null");
  if (m == 0 || k == 0 || k % 256 != 0 || k > 4096)
    return fail(AIMA_MOE_ERR_UNSUPPORTED, "gemv needs k a multiple of 256 up to 4096 and m > 0");
  const cudaError_t error = launch_gemv_bf16(weight, x, out, static_cast<int>(m),
                                             static_cast<int>(k), static_cast<cudaStream_t>(stream));
  if (error != cudaSuccess) return fail_cuda(error, "launch gemv_bf16_kernel");
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_gemm_bf16_launch(aima_moe_handle* handle, const void* a, const void* b,
                                          void* d, uint32_t m, uint32_t n, uint32_t k, void* stream) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if (const int wrong_device = check_current_device(handle); wrong_device != AIMA_MOE_OK) return wrong_device;
  if (a == nullptr || b == nullptr || d == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "gemm pointer is null");
  if (m == 0 || n == 0 || k == 0 || k % 64 != 0 || n % 8 != 0)
    return fail(AIMA_MOE_ERR_UNSUPPORTED, "gemm needs k a multiple of 64 and n a multiple of 8");
  GroupedGemm g{};
  g.max_tiles = static_cast<int>((m + kTileRows - 1) / kTileRows);
  g.dense_rows = static_cast<int>(m);
  g.a = static_cast<const __nv_bfloat16*>(a); g.lda = static_cast<int>(k); g.k = static_cast<int>(k);
  g.b0 = static_cast<const __nv_bfloat16*>(b);
  g.n = static_cast<int>(n);
  g.c = static_cast<__nv_bfloat16*>(d); g.ldc = static_cast<int>(n);
  TcExtra extra{};
  extra.status = handle->status; extra.sm_count = handle->sm_count; extra.a_rows = m; extra.experts_in_b = 1;
  const cudaError_t error = launch_grouped_gemm_tc(kGemmPlain, g, extra, static_cast<cudaStream_t>(stream));
  if (error != cudaSuccess) return fail_cuda(error, "launch grouped_gemm_tc_kernel (plain)");
  handle->last_stream = static_cast<cudaStream_t>(stream);
  handle->metrics.kernel_launches += 1;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_sync_metrics(aima_moe_handle* handle, aima_moe_metrics* metrics) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  cudaError_t error = cudaStreamSynchronize(handle->last_stream);
  if (error != cudaSuccess) return fail_cuda(error, "cudaStreamSynchronize");
  int status_words[24] = {};
  error = cudaMemcpy(status_words, handle->status, sizeof status_words, cudaMemcpyDeviceToHost);
  if (error != cudaSuccess) return fail_cuda(error, "cudaMemcpy status word");
  const int device_status = status_words[0];
  handle->metrics.device_status = device_status;
  if (handle->prefill.total_bytes != 0) {
    error = cudaMemcpy(&handle->metrics.last_padded_routed_rows, handle->prefill.padded_rows,
                       sizeof(int32_t), cudaMemcpyDeviceToHost);
    if (error != cudaSuccess) return fail_cuda(error, "cudaMemcpy padded row count");
    int32_t stats[5] = {0, 0, 0, 0, 0};
    error = cudaMemcpy(stats, handle->prefill.router_stats, sizeof stats, cudaMemcpyDeviceToHost);
    if (error != cudaSuccess) return fail_cuda(error, "cudaMemcpy router statistics");
    handle->metrics.router_candidates = static_cast<uint64_t>(static_cast<uint32_t>(stats[0]));
    handle->metrics.router_tokens = static_cast<uint64_t>(static_cast<uint32_t>(stats[1]));
    handle->metrics.router_bound_violations = static_cast<uint64_t>(static_cast<uint32_t>(stats[2]));
    handle->metrics.router_audited_tokens = static_cast<uint64_t>(static_cast<uint32_t>(stats[3]));
    handle->metrics.router_audit_mismatches = static_cast<uint64_t>(static_cast<uint32_t>(stats[4]));
  }
  if (metrics != nullptr) {
    if (metrics->struct_bytes != sizeof(aima_moe_metrics))
      return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "aima_moe_metrics size mismatch");
    *metrics = handle->metrics;
  }
  if (device_status != 0) {
    const int reset = reset_decode_sync(handle);
    if (reset != AIMA_MOE_OK) return reset;
    return fail(AIMA_MOE_ERR_TIMEOUT,
                "a bounded device-side wait ran out (status %d, site %d, block %d, warp %d, detail %d, "
                "spins %d, elapsed_us %d, barrier %08x:%08x); sync state reset",
                device_status, status_words[1], status_words[2], status_words[3], status_words[4],
                status_words[5], status_words[6], static_cast<unsigned>(status_words[8]),
                static_cast<unsigned>(status_words[7]));
  }
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_ep_local_buffer(aima_moe_handle* handle, void** pointer, uint64_t* bytes) {
  if (handle == nullptr || pointer == nullptr || bytes == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "expert-parallel buffer argument is null");
  if (handle->ep_local == nullptr)
    return fail(AIMA_MOE_ERR_UNSUPPORTED, "the handle was prepared with world = 1");
  *pointer = handle->ep_local;
  *bytes = handle->ep_bytes;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_ep_export(aima_moe_handle* handle, void* ipc_handle_64_bytes) {
  if (handle == nullptr || ipc_handle_64_bytes == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "expert-parallel export argument is null");
  if (handle->ep_local == nullptr)
    return fail(AIMA_MOE_ERR_UNSUPPORTED, "the handle was prepared with world = 1");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t ipc;
  const cudaError_t error = cudaIpcGetMemHandle(&ipc, handle->ep_local);
  if (error != cudaSuccess) return fail_cuda(error, "cudaIpcGetMemHandle");
  std::memcpy(ipc_handle_64_bytes, &ipc, sizeof ipc);
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_ep_connect(aima_moe_handle* handle, uint32_t peer, const void* ipc_handle_64_bytes,
                                    void* direct_pointer) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if (handle->ep_local == nullptr)
    return fail(AIMA_MOE_ERR_UNSUPPORTED, "the handle was prepared with world = 1");
  if (peer >= handle->config.world)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "peer %u is not a rank of world %u", peer, handle->config.world);
  if ((ipc_handle_64_bytes == nullptr) == (direct_pointer == nullptr))
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "give exactly one of an IPC handle or a direct device pointer");
  // peer == rank with a direct pointer substitutes this rank's own buffer (hosts that own a
  // symmetric heap); an IPC handle for oneself makes no sense
  if (peer == handle->config.rank && direct_pointer == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "the own rank can only be given as a direct pointer");
  if (direct_pointer != nullptr) {
    handle->ep_peers[peer] = static_cast<unsigned long long*>(direct_pointer);
    return AIMA_MOE_OK;
  }
  cudaIpcMemHandle_t ipc;
  std::memcpy(&ipc, ipc_handle_64_bytes, sizeof ipc);
  void* mapped = nullptr;
  const cudaError_t error = cudaIpcOpenMemHandle(&mapped, ipc, cudaIpcMemLazyEnablePeerAccess);
  if (error != cudaSuccess) return fail_cuda(error, "cudaIpcOpenMemHandle");
  handle->ep_ipc_opened[peer] = mapped;
  handle->ep_peers[peer] = static_cast<unsigned long long*>(mapped);
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_debug_set_decode_epoch(aima_moe_handle* handle, uint32_t epoch) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if (const int wrong_device = check_current_device(handle); wrong_device != AIMA_MOE_OK) return wrong_device;
  // after everything enqueued so far: the kernels read the word when they start
  epoch %= kDecodeEpochPeriod;
  cudaError_t error = cudaDeviceSynchronize();
  if (error == cudaSuccess) error = cudaMemcpy(handle->epoch_base, &epoch, sizeof epoch, cudaMemcpyHostToDevice);
  if (error != cudaSuccess) return fail_cuda(error, "cudaMemcpy decode epoch");
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_set_tracing(aima_moe_handle* handle, int enabled) {
  if (handle == nullptr) return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  handle->tracing = enabled != 0;
  handle->traced_layers = 0;
  handle->ep_prefill.trace = handle->tracing;
  if (handle->tracing && handle->config.world > 1 && handle->ep_prefill.stage_events[0] == nullptr) {
    for (int i = 0; i <= kEpPrefillStages; ++i) {
      const cudaError_t error = cudaEventCreate(&handle->ep_prefill.stage_events[i]);
      if (error != cudaSuccess) return fail_cuda(error, "cudaEventCreate prefill stage event");
    }
  }
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_read_decode_timeline(aima_moe_handle* handle, uint64_t* stamps_ns,
                                              uint32_t capacity, uint32_t* written) {
  if (handle == nullptr || stamps_ns == nullptr || written == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "timeline argument is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  const uint32_t layers = handle->traced_layers < capacity / kDecodeTraceStamps ? handle->traced_layers
                                                                               : capacity / kDecodeTraceStamps;
  cudaError_t error = cudaStreamSynchronize(handle->last_stream);
  if (error != cudaSuccess) return fail_cuda(error, "cudaStreamSynchronize");
  if (layers != 0) {
    // block 0's record: kDecodeTraceSlots words per layer, of which the first kDecodeTraceStamps are returned
    error = cudaMemcpy2D(stamps_ns, sizeof(uint64_t) * kDecodeTraceStamps, handle->timeline,
                         sizeof(uint64_t) * kDecodeTraceSlots, sizeof(uint64_t) * kDecodeTraceStamps, layers,
                         cudaMemcpyDeviceToHost);
    if (error != cudaSuccess) return fail_cuda(error, "cudaMemcpy decode timeline");
  }
  *written = layers * kDecodeTraceStamps;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_read_decode_block_timelines(aima_moe_handle* handle, uint64_t* stamps_ns,
                                                     uint32_t capacity, uint32_t* blocks, uint32_t* layers) {
  if (handle == nullptr || stamps_ns == nullptr || blocks == nullptr || layers == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "timeline argument is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  const uint32_t n_blocks = static_cast<uint32_t>(handle->decode_grid);
  const uint32_t n_layers = handle->traced_layers;
  if (static_cast<uint64_t>(n_blocks) * n_layers * kDecodeTraceSlots > capacity)
    return fail(AIMA_MOE_ERR_CAPACITY, "timeline buffer holds %u words, %u blocks x %u layers x %d are needed",
                capacity, n_blocks, n_layers, kDecodeTraceSlots);
  cudaError_t error = cudaStreamSynchronize(handle->last_stream);
  if (error != cudaSuccess) return fail_cuda(error, "cudaStreamSynchronize");
  if (n_layers != 0) {
    error = cudaMemcpy2D(stamps_ns, sizeof(uint64_t) * kDecodeTraceSlots * n_layers, handle->timeline,
                         sizeof(uint64_t) * kDecodeTraceSlots * kMaxLayers,
                         sizeof(uint64_t) * kDecodeTraceSlots * n_layers, n_blocks, cudaMemcpyDeviceToHost);
    if (error != cudaSuccess) return fail_cuda(error, "cudaMemcpy decode block timelines");
  }
  *blocks = n_blocks;
  *layers = n_layers;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_read_ep_prefill_stages(aima_moe_handle* handle, float* stage_ms, uint32_t capacity,
                                                uint32_t* written) {
  if (handle == nullptr || stage_ms == nullptr || written == nullptr)
    return fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "stage timing argument is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  *written = 0;
  if (!handle->ep_prefill.trace || handle->ep_prefill.stage_events[0] == nullptr || handle->ep_prefill.epoch == 0)
    return AIMA_MOE_OK;
  cudaError_t error = cudaStreamSynchronize(handle->last_stream);
  if (error != cudaSuccess) return fail_cuda(error, "cudaStreamSynchronize");
  for (uint32_t i = 0; i < static_cast<uint32_t>(kEpPrefillStages) && i < capacity; ++i) {
    error = cudaEventElapsedTime(stage_ms + i, handle->ep_prefill.stage_events[i],
                                 handle->ep_prefill.stage_events[i + 1]);
    if (error != cudaSuccess) return fail_cuda(error, "cudaEventElapsedTime prefill stage");
    *written = i + 1;
  }
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_release(aima_moe_handle* handle) {
  if (handle == nullptr) return AIMA_MOE_OK;
  for (int i = 0; i < 8; ++i) {
    if (handle->ep_prefill.stage_events[i] != nullptr) cudaEventDestroy(handle->ep_prefill.stage_events[i]);
  }
  for (int peer = 0; peer < 8; ++peer) {
    if (handle->ep_ipc_opened[peer] != nullptr) cudaIpcCloseMemHandle(handle->ep_ipc_opened[peer]);
  }
  cudaFree(handle->ep_local);
  cudaFree(handle->timeline);
  cudaFree(handle->router_row_norms);
  cudaFree(handle->dev_layers);
  cudaFree(handle->decode_scratch);
  prefill_workspace_free(&handle->prefill);
  delete handle;
  return AIMA_MOE_OK;
}

}  // extern "C"
