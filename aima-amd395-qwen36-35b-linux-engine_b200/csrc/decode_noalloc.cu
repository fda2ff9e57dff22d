// Allocation-free decode entry point.
//
// Some hosts cannot let a provider allocate device memory: a serving process
// that has already handed every free byte of HBM to its own weight and KV-cache
// arenas (a later cudaMalloc would fail or fragment them), or a request path
// that must never reach an allocating call because cudaMalloc / cudaFree
// synchronise the whole device and stall the streams of the request in flight.
// aima_moe_prepare() allocates, so such hosts cannot use the handle-based API.
// This entry point needs no handle: the few kilobytes the persistent decode
// kernel needs besides its inputs and outputs (layer table, inter-layer
// vectors, router logits, activations, grid-barrier words, status word) live in
// one file-scope __device__ array that every GPU loading this library holds
// until the process exits.
#include "../../include/aima_moe.h"

#include "decode_kernel.cuh"

#include <cstdio>
#include <mutex>

namespace aima {
void set_last_error_message(const char* message);   // defined next to aima_moe_last_error_string
}
using namespace aima;

namespace {

constexpr int kNoAllocMaxDevices = 64;

// layout of the static scratch array (bytes)
constexpr size_t kOffTable = 0;                                   // LayerPtrs[AIMA_MOE_NOALLOC_MAX_LAYERS]
constexpr size_t kOffSync = 1024;                                 // barrier counter (+0), base (+128), tag base (+192)
constexpr size_t kOffStatus = kOffSync + 256;                     // device status words
constexpr size_t kOffLogits = kOffStatus + 256;                   // replicated tagged 64-bit router logits
constexpr size_t kOffX0 = kOffLogits + static_cast<size_t>(kDecodeLogitWords) * 8;            // tagged vector 0
constexpr size_t kOffX1 = kOffX0 + static_cast<size_t>(kDecodeReplicas) * kHidden * 4;        // tagged vector 1
constexpr size_t kOffAct = kOffX1 + static_cast<size_t>(kDecodeReplicas) * kHidden * 4;       // activation copies
constexpr size_t kClearBytes = kOffAct - kOffSync;                // everything that carries a tag or a count
constexpr size_t kScratchBytes = kOffAct + static_cast<size_t>(kDecodeReplicas) * kDecodeActStride * 4;
static_assert(sizeof(LayerPtrs) * AIMA_MOE_NOALLOC_MAX_LAYERS <= kOffSync - kOffTable, "layer table overflows its slot");
static_assert(kScratchBytes <= AIMA_MOE_NOALLOC_SCRATCH_BYTES, "scratch exceeds the stated maximum");

// In host code this name is only a stand-in for the device array; its device
// address comes from cudaGetSymbolAddress (see scratch_for_current_device).
static __device__ __align__(256) unsigned char g_noalloc_scratch[AIMA_MOE_NOALLOC_SCRATCH_BYTES];

struct LayerTable {
  LayerPtrs entry[AIMA_MOE_NOALLOC_MAX_LAYERS];
};

// Device code may name the array directly.
__global__ void noalloc_write_layer_table_kernel(const LayerTable table, int n_layers) {
  LayerPtrs* slots = reinterpret_cast<LayerPtrs*>(g_noalloc_scratch + kOffTable);
  const int i = threadIdx.x;
  if (i < n_layers) slots[i] = table.entry[i];
}

std::mutex g_setup_mutex;
unsigned char* g_device_scratch[kNoAllocMaxDevices] = {};
int g_device_grid[kNoAllocMaxDevices] = {};

int noalloc_fail(int code, const char* message) {
  set_last_error_message(message);   // read back with aima_moe_last_error_string()
  return code;
}

// One-time set-up for the current device: resolve the device address of the
// static array and check that the device can run the cooperative kernel.
int scratch_for_current_device(unsigned char** scratch, int* grid) {
  int device = -1;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) {
    (void)cudaGetLastError();
    return noalloc_fail(AIMA_MOE_ERR_NO_DEVICE, "no CUDA device is current");
  }
  if (device < 0 || device >= kNoAllocMaxDevices)
    return noalloc_fail(AIMA_MOE_ERR_UNSUPPORTED, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_device_scratch[device] == nullptr) {
    int major = 0, sm_count = 0, cooperative = 0;
    error = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (error == cudaSuccess) error = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    if (error == cudaSuccess) error = cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device);
    if (error != cudaSuccess) {
      (void)cudaGetLastError();
      return noalloc_fail(static_cast<int>(error), "cudaDeviceGetAttribute failed");
    }
    if (major != 10) return noalloc_fail(AIMA_MOE_ERR_NO_DEVICE, "device is not an sm_100 part");
    const int blocks = sm_count < kDecodeMaxBlocks ? sm_count : kDecodeMaxBlocks;
    if (blocks < kDecodeMinBlocks || !cooperative)
      return noalloc_fail(AIMA_MOE_ERR_UNSUPPORTED, "device cannot run the cooperative decode kernel");
    unsigned char* pointer = nullptr;
    error = cudaGetSymbolAddress(reinterpret_cast<void**>(&pointer), g_noalloc_scratch);
    if (error != cudaSuccess || pointer == nullptr) {
      (void)cudaGetLastError();
      return noalloc_fail(error != cudaSuccess ? static_cast<int>(error) : AIMA_MOE_ERR_INTERNAL,
                          "cudaGetSymbolAddress(static decode scratch) failed");
    }
    g_device_scratch[device] = pointer;
    g_device_grid[device] = blocks;
  }
  *scratch = g_device_scratch[device];
  *grid = g_device_grid[device];
  return AIMA_MOE_OK;
}

// Null, size and alignment first; then residency: the kernel reads these pointers with bulk copies
// and plain loads, so host memory or another GPU's memory must be turned away here, on the host,
// with an error code -- not met on the device as a fault.  cudaPointerGetAttributes allocates nothing.
bool resident_on(const void* pointer, int device) {
  cudaPointerAttributes attributes{};
  if (cudaPointerGetAttributes(&attributes, pointer) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  if (attributes.type == cudaMemoryTypeManaged) return true;
  return attributes.type == cudaMemoryTypeDevice && attributes.device == device;
}
bool tensor_ok(const void* pointer, uint64_t bytes, uint64_t expected, int device) {
  return pointer != nullptr && bytes == expected && reinterpret_cast<uintptr_t>(pointer) % 16 == 0 &&
         resident_on(pointer, device);
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int aima_moe_decode_layers_noalloc(const aima_moe_layer_weights* layers, uint32_t n_layers,
                                   const void* x_in, void* x_out, float rms_eps,
                                   int32_t* device_status, void* stream) {
  if (layers == nullptr || x_in == nullptr || x_out == nullptr)
    return noalloc_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "layers, x_in and x_out must not be null");
  if (n_layers == 0)
    return noalloc_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "n_layers is zero");
  if (n_layers > AIMA_MOE_NOALLOC_MAX_LAYERS)
    return noalloc_fail(AIMA_MOE_ERR_CAPACITY,
                        "n_layers exceeds AIMA_MOE_NOALLOC_MAX_LAYERS: the static scratch holds at most "
                        "8 layer entries; split the call or use the handle-based API");
  if (!(rms_eps > 0.0f) || !(rms_eps < 1.0f))
    return noalloc_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "rms_eps must be in (0, 1)");
  const uintptr_t in0 = reinterpret_cast<uintptr_t>(x_in), out0 = reinterpret_cast<uintptr_t>(x_out);
  if (in0 % 16 != 0 || out0 % 16 != 0)
    return noalloc_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "x_in and x_out must be 16-byte aligned");
  if (in0 < out0 + kHidden * 2 && out0 < in0 + kHidden * 2)
    return noalloc_fail(AIMA_MOE_ERR_ALIAS, "x_out aliases x_in");

  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) {
    (void)cudaGetLastError();
    return noalloc_fail(AIMA_MOE_ERR_NO_DEVICE, "no CUDA device is current");
  }
  if (!tensor_ok(x_in, kHidden * 2, kHidden * 2, device) || !tensor_ok(x_out, kHidden * 2, kHidden * 2, device))
    return noalloc_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "x_in and x_out must be memory of the current device");
  if (device_status != nullptr && !resident_on(device_status, device))
    return noalloc_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "device_status must be memory of the current device");

  LayerTable table{};
  for (uint32_t i = 0; i < n_layers; ++i) {
    const aima_moe_layer_weights& w = layers[i];
    if (w.struct_bytes != sizeof(aima_moe_layer_weights))
      return noalloc_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "aima_moe_layer_weights size mismatch");
    const bool ok =
        tensor_ok(w.router, w.router_bytes, 2ull * kExperts * kHidden, device) &&
        tensor_ok(w.expert_gate_up, w.expert_gate_up_bytes, 2ull * kExperts * 2 * kInter * kHidden, device) &&
        tensor_ok(w.expert_down, w.expert_down_bytes, 2ull * kExperts * kHidden * kInter, device) &&
        tensor_ok(w.shared_expert_gate, w.shared_expert_gate_bytes, 2ull * kHidden, device) &&
        tensor_ok(w.shared_gate_proj, w.shared_gate_proj_bytes, 2ull * kSharedInter * kHidden, device) &&
        tensor_ok(w.shared_up_proj, w.shared_up_proj_bytes, 2ull * kSharedInter * kHidden, device) &&
        tensor_ok(w.shared_down_proj, w.shared_down_proj_bytes, 2ull * kHidden * kSharedInter, device) &&
        tensor_ok(w.post_attention_norm, w.post_attention_norm_bytes, 2ull * kHidden, device);
    if (!ok)
      return noalloc_fail(AIMA_MOE_ERR_INVALID_ARGUMENT,
                          "a layer tensor is null, misaligned, not memory of the current device or has the "
                          "wrong byte size (all 256 experts and the norm weight are required)");
    LayerPtrs& e = table.entry[i];
    e.router = static_cast<const __nv_bfloat16*>(w.router);
    e.expert_gate_up = static_cast<const __nv_bfloat16*>(w.expert_gate_up);
    e.expert_down = static_cast<const __nv_bfloat16*>(w.expert_down);
    e.shared_gate = static_cast<const __nv_bfloat16*>(w.shared_expert_gate);
    e.shared_gate_proj = static_cast<const __nv_bfloat16*>(w.shared_gate_proj);
    e.shared_up_proj = static_cast<const __nv_bfloat16*>(w.shared_up_proj);
    e.shared_down_proj = static_cast<const __nv_bfloat16*>(w.shared_down_proj);
    e.norm_weight = static_cast<const __nv_bfloat16*>(w.post_attention_norm);
  }

  unsigned char* scratch = nullptr;
  int grid = 0;
  const int setup = scratch_for_current_device(&scratch, &grid);
  if (setup != AIMA_MOE_OK) return setup;
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);

  // The array keeps whatever the previous call left.  The barrier words, the
  // status word and every tagged exchange word (their tags restart with each
  // call) must start at zero; everything else is written before it is read.
  cudaError_t error = cudaMemsetAsync(scratch + kOffSync, 0, kClearBytes, cuda_stream);
  if (error != cudaSuccess) {
    (void)cudaGetLastError();
    return noalloc_fail(static_cast<int>(error), "cudaMemsetAsync(static scratch sync words) failed");
  }
  noalloc_write_layer_table_kernel<<<1, 32, 0, cuda_stream>>>(table, static_cast<int>(n_layers));
  error = cudaGetLastError();
  if (error != cudaSuccess)
    return noalloc_fail(static_cast<int>(error), "launch of the layer-table kernel failed");

  DecodeParams params{};
  params.layers = reinterpret_cast<const LayerPtrs*>(scratch + kOffTable);
  params.x_in = static_cast<const __nv_bfloat16*>(x_in);
  params.x_out = static_cast<__nv_bfloat16*>(x_out);
  params.xbuf0 = reinterpret_cast<uint32_t*>(scratch + kOffX0);
  params.xbuf1 = reinterpret_cast<uint32_t*>(scratch + kOffX1);
  params.logits = reinterpret_cast<unsigned long long*>(scratch + kOffLogits);
  params.act = reinterpret_cast<uint32_t*>(scratch + kOffAct);
  params.epoch_base = reinterpret_cast<unsigned*>(scratch + kOffSync + 192);
  params.status = reinterpret_cast<int*>(scratch + kOffStatus);
  params.router_bias = nullptr;
  params.timeline = nullptr;
  params.world = 1;
  params.rank = 0;
  params.quant_eighths = 0;
  params.speculate = 1;
  params.max_in_flight = kDecodeDefaultInFlight;
  params.eps = rms_eps;
  params.first_layer = 0;
  params.n_layers = static_cast<int>(n_layers);
  params.expert_lo = 0;
  params.expert_hi = kExperts;
  error = launch_moe_decode(params, grid, cuda_stream);
  if (error != cudaSuccess) {
    (void)cudaGetLastError();
    return noalloc_fail(static_cast<int>(error), "launch of the persistent decode kernel failed");
  }
  if (device_status != nullptr) {
    error = cudaMemcpyAsync(device_status, scratch + kOffStatus, sizeof(int32_t),
                            cudaMemcpyDeviceToDevice, cuda_stream);
    if (error != cudaSuccess) {
      (void)cudaGetLastError();
      return noalloc_fail(static_cast<int>(error), "cudaMemcpyAsync(status word) failed");
    }
  }
  return AIMA_MOE_OK;
}
