// Row-wise helpers around the MoE half-layer: residual add + RMSNorm and a
// batch-1 BF16 GEMV.
//
// RMSNorm follows prefill_rmsnorm_2048_kernel / prefill_add_rmsnorm_2048_kernel
// (native/src/native_pointwise.hip.cpp:109-182): optional r = bf16(x + residual),
// out = bf16(r * rsqrt(mean(r^2) + eps) * (weight + 1)) with the correctly
// rounded reciprocal square root (:37-69).  The GEMV has the contract of
// launch_bf16_wvsplitk (native/src/bf16_wvsplitk.hip.cpp:337-366):
// out[m] = bf16(x . W[m, :]), FP32 accumulation.
#include "pointwise.cuh"

namespace aima {
namespace {

constexpr int kNormWarpsPerBlock = 8;

// One warp per row.  Lane l holds elements 256 g + 8 l + j (g, j in 0..7) in
// v[8 g + j]; the sum of squares follows the reference kernel's order
// (row_sumsq_2048 in common.cuh).
__global__ void __launch_bounds__(kNormWarpsPerBlock * 32)
rmsnorm_rows_kernel(const __nv_bfloat16* __restrict__ x,
                    const __nv_bfloat16* __restrict__ residual,
                    const __nv_bfloat16* __restrict__ weight,
                    __nv_bfloat16* __restrict__ residual_out,
                    __nv_bfloat16* __restrict__ norm_out, int rows, float eps) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a product kernel that follows may set itself up
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kNormWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= rows) return;
  const size_t base = static_cast<size_t>(row) * kHidden;
  float v[64];
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const size_t off = base + 256 * g + 8 * lane;
    const uint4 xv = *reinterpret_cast<const uint4*>(x + off);
    unpack8(xv, v + 8 * g);
    if (residual != nullptr) {
      float r[8];
      unpack8(*reinterpret_cast<const uint4*>(residual + off), r);
      uint32_t packed[4];
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const uint16_t lo = float_to_bf16_bits(__fadd_rn(v[8 * g + j], r[j]));
        const uint16_t hi = float_to_bf16_bits(__fadd_rn(v[8 * g + j + 1], r[j + 1]));
        v[8 * g + j] = bf16_bits_to_float(lo);
        v[8 * g + j + 1] = bf16_bits_to_float(hi);
        packed[j / 2] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
      }
      if (residual_out != nullptr) {
        *reinterpret_cast<uint4*>(residual_out + off) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
  }
  const float total = row_sumsq_2048(v, lane);
  const float inv = det_rsqrtf(__fadd_rn(__fdiv_rn(total, static_cast<float>(kHidden)), eps));
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    float w[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(weight) + g * 32 + lane), w);
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const float a = __fmul_rn(__fmul_rn(v[8 * g + j], inv), __fadd_rn(w[j], 1.0f));
      const float b = __fmul_rn(__fmul_rn(v[8 * g + j + 1], inv), __fadd_rn(w[j + 1], 1.0f));
      packed[j / 2] = static_cast<uint32_t>(float_to_bf16_bits(a)) |
                      (static_cast<uint32_t>(float_to_bf16_bits(b)) << 16);
    }
    *reinterpret_cast<uint4*>(norm_out + base + 256 * g + 8 * lane) =
        make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

// One warp per output row; K is a multiple of 256 and at most 4096.
constexpr int kGemvWarpsPerBlock = 8;
__global__ void __launch_bounds__(kGemvWarpsPerBlock * 32)
gemv_bf16_kernel(const __nv_bfloat16* __restrict__ weight,
                 const __nv_bfloat16* __restrict__ x,
                 __nv_bfloat16* __restrict__ out, int m, int k) {
  __shared__ __align__(16) uint16_t xs[4096];
  for (int v = threadIdx.x; v < k / 8; v += blockDim.x) {
    reinterpret_cast<uint4*>(xs)[v] = reinterpret_cast<const uint4*>(x)[v];
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kGemvWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= m) return;
  const uint4* wrow = reinterpret_cast<const uint4*>(weight + static_cast<size_t>(row) * k) + lane;
  const uint4* xrow = reinterpret_cast<const uint4*>(xs) + lane;
  float acc = 0.0f;
  for (int i = 0; i < k / 256; ++i) {
    float xf[8];
    unpack8(xrow[i * 32], xf);
    acc = fma8(xf, wrow[i * 32], acc);
  }
  acc = butterfly_sum(acc);
  if (lane == 0) out[row] = __float2bfloat16_rn(acc);
}

}  // namespace

cudaError_t launch_rmsnorm_rows(const void* x, const void* residual,
                                const void* weight, void* residual_out,
                                void* norm_out, int rows, float eps,
                                cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  const int blocks = (rows + kNormWarpsPerBlock - 1) / kNormWarpsPerBlock;
  rmsnorm_rows_kernel<<<blocks, kNormWarpsPerBlock * 32, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(residual),
      static_cast<const __nv_bfloat16*>(weight),
      static_cast<__nv_bfloat16*>(residual_out),
      static_cast<__nv_bfloat16*>(norm_out), rows, eps);
  return cudaGetLastError();
}

cudaError_t launch_gemv_bf16(const void* weight, const void* x, void* out,
                             int m, int k, cudaStream_t stream) {
  const int blocks = (m + kGemvWarpsPerBlock - 1) / kGemvWarpsPerBlock;
  gemv_bf16_kernel<<<blocks, kGemvWarpsPerBlock * 32, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(weight),
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), m, k);
  return cudaGetLastError();
}

}  // namespace aima
