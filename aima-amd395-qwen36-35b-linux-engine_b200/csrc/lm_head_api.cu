// C ABI of the LM head with a certified top-1 (declarations and contract in include/aima_moe.h).
#include "lm_head.cuh"

#include <cstdio>
#include <mutex>
#include <new>

struct aima_moe_lm_head {
  std::mutex mutex;
  int device = 0;
  int sm_count = 0;
  uint32_t rows = 0;
  const void* weight = nullptr;      // caller-owned raw BF16 matrix [rows, 2048]
  void* allocation = nullptr;        // q | scales | residual_l2 | wire | partial | candidate ids
  aima::LmHeadBuffers buffers{};
  cudaStream_t last_stream = nullptr;
  uint64_t launches = 0;
};

namespace aima {
void set_last_error_message(const char* message);
}

namespace {

int lm_fail(int status, const char* message) {
  aima::set_last_error_message(message);
  return status;
}

int lm_fail_cuda(cudaError_t error, const char* what) {
  char text[256];
  std::snprintf(text, sizeof text, "%s: %s", what, cudaGetErrorString(error));
  aima::set_last_error_message(text);
  (void)cudaGetLastError();
  return static_cast<int>(error);
}

size_t align256(size_t bytes) { return (bytes + 255) / 256 * 256; }

}  // namespace

extern "C" {

#define AIMA_EXPORT __attribute__((visibility("default")))

AIMA_EXPORT int aima_moe_lm_head_build(const void* weight_bf16, uint32_t rows, aima_moe_lm_head** out,
                                       void* stream) {
  if (out == nullptr) return lm_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "lm head: out is null");
  *out = nullptr;
  if (weight_bf16 == nullptr || rows == 0 || rows > (1u << 24))
    return lm_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "lm head: weight is null or rows outside 1 .. 2^24");
  if (reinterpret_cast<uintptr_t>(weight_bf16) % 16 != 0)
    return lm_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "lm head: weight is not 16-byte aligned");
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) {
    (void)cudaGetLastError();
    return lm_fail(AIMA_MOE_ERR_NO_DEVICE, "lm head: no CUDA device (there is no CPU fallback)");
  }
  cudaDeviceProp properties{};
  error = cudaGetDeviceProperties(&properties, device);
  if (error != cudaSuccess) return lm_fail_cuda(error, "cudaGetDeviceProperties");
  if (properties.major != 10)
    return lm_fail(AIMA_MOE_ERR_NO_DEVICE, "lm head: needs an sm_100 device");
  cudaPointerAttributes attributes{};
  error = cudaPointerGetAttributes(&attributes, weight_bf16);
  if (error != cudaSuccess) return lm_fail_cuda(error, "cudaPointerGetAttributes");
  if (attributes.type != cudaMemoryTypeDevice && attributes.type != cudaMemoryTypeManaged)
    return lm_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "lm head: weight is not device resident");

  aima_moe_lm_head* handle = new (std::nothrow) aima_moe_lm_head();
  if (handle == nullptr) return lm_fail(AIMA_MOE_ERR_INTERNAL, "lm head: out of host memory");
  handle->device = device;
  handle->sm_count = properties.multiProcessorCount;
  handle->rows = rows;
  handle->weight = weight_bf16;
  const size_t q_bytes = align256(static_cast<size_t>(rows) * aima::kHidden);
  const size_t row_bytes = align256(static_cast<size_t>(rows) * sizeof(float));
  const size_t total = q_bytes + 2 * row_bytes + 256 + 1024 +
                       align256(AIMA_MOE_LM_HEAD_CANDIDATES * sizeof(uint32_t));
  error = cudaMalloc(&handle->allocation, total);
  if (error != cudaSuccess) {
    delete handle;
    return lm_fail_cuda(error, "cudaMalloc lm head");
  }
  uint8_t* cursor = static_cast<uint8_t*>(handle->allocation);
  handle->buffers.q_weight = reinterpret_cast<int8_t*>(cursor); cursor += q_bytes;
  handle->buffers.scales = reinterpret_cast<float*>(cursor); cursor += row_bytes;
  handle->buffers.residual_l2 = reinterpret_cast<float*>(cursor); cursor += row_bytes;
  handle->buffers.wire = reinterpret_cast<aima_moe_lm_head_result*>(cursor); cursor += 256;
  handle->buffers.partial = reinterpret_cast<float*>(cursor); cursor += 1024;
  handle->buffers.candidate_ids = reinterpret_cast<uint32_t*>(cursor);
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  error = cudaMemsetAsync(handle->buffers.wire, 0, 256, cuda_stream);
  if (error == cudaSuccess)
    error = aima::lm_head_quantize(weight_bf16, static_cast<int>(rows), handle->buffers.q_weight,
                                   handle->buffers.scales, handle->buffers.residual_l2, cuda_stream);
  if (error != cudaSuccess) {
    cudaFree(handle->allocation);
    delete handle;
    return lm_fail_cuda(error, "lm head quantisation");
  }
  handle->last_stream = cuda_stream;
  handle->launches = 1;
  *out = handle;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_lm_head_views(aima_moe_lm_head* handle, void** q_weight, void** scales,
                                       void** residual_l2) {
  if (handle == nullptr) return lm_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "lm head: handle is null");
  if (q_weight != nullptr) *q_weight = handle->buffers.q_weight;
  if (scales != nullptr) *scales = handle->buffers.scales;
  if (residual_l2 != nullptr) *residual_l2 = handle->buffers.residual_l2;
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_lm_head_launch(aima_moe_lm_head* handle, const void* hidden_bf16, void* logits_f32,
                                        void* stream) {
  if (handle == nullptr) return lm_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "lm head: handle is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  if (hidden_bf16 == nullptr || logits_f32 == nullptr)
    return lm_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "lm head: hidden or logits is null");
  if (reinterpret_cast<uintptr_t>(hidden_bf16) % 16 != 0 || reinterpret_cast<uintptr_t>(logits_f32) % 16 != 0)
    return lm_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "lm head: hidden and logits must be 16-byte aligned");
  int launches = 0;
  const cudaError_t error =
      aima::lm_head_certify(handle->buffers, handle->weight, hidden_bf16, static_cast<float*>(logits_f32),
                            static_cast<int>(handle->rows), handle->sm_count,
                            static_cast<cudaStream_t>(stream), &launches);
  if (error != cudaSuccess) return lm_fail_cuda(error, "lm head launch");
  handle->last_stream = static_cast<cudaStream_t>(stream);
  handle->launches += static_cast<uint64_t>(launches);
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_lm_head_read_result(aima_moe_lm_head* handle, aima_moe_lm_head_result* result) {
  if (handle == nullptr || result == nullptr)
    return lm_fail(AIMA_MOE_ERR_INVALID_ARGUMENT, "lm head: handle or result is null");
  std::lock_guard<std::mutex> lock(handle->mutex);
  cudaError_t error = cudaStreamSynchronize(handle->last_stream);
  if (error != cudaSuccess) return lm_fail_cuda(error, "cudaStreamSynchronize");
  error = cudaMemcpy(result, handle->buffers.wire, sizeof *result, cudaMemcpyDeviceToHost);
  if (error != cudaSuccess) return lm_fail_cuda(error, "cudaMemcpy lm head result");
  if (result->overflow != 0)
    return lm_fail(AIMA_MOE_ERR_CAPACITY, "lm head: more than 1024 candidates, the top-1 is not certified");
  return AIMA_MOE_OK;
}

AIMA_EXPORT int aima_moe_lm_head_release(aima_moe_lm_head* handle) {
  if (handle == nullptr) return AIMA_MOE_OK;
  cudaFree(handle->allocation);
  delete handle;
  return AIMA_MOE_OK;
}

}  // extern "C"
