// LM head with a certified top-1: a row-wise int8 copy of the vocabulary matrix is scanned for
// every token (one byte per weight instead of two), Cauchy-Schwarz bounds around the approximate
// logits decide which rows can still win, and only those are evaluated exactly in BF16.
//
// Follows NativeLmHeadStore::build / quantize_lm_head_rowwise_kernel
// (native/src/native_lm_head.hip.cpp:53-115, 126-176), the row-wise int8 GEMV of
// benchmarks/shape-lab/four_layer_mini_engine.py:1223-1258 and launch_native_lm_head_certificate
// (native/src/native_lm_head_certificate.hip.cpp:44-275): same bounds, same outward rounding,
// same capacity of 1024 candidates, same tie rule (equal logits -> lowest token id).
// The scan is the bandwidth-bound kernel: rows x 2048 bytes per token.
#include "lm_head.cuh"

#include <math_constants.h>

namespace aima {
namespace {

constexpr int kLmThreads = 256;
constexpr int kLmBoundBlocks = 256;
constexpr int kResidualSafetyUlps = 8;
constexpr int kHiddenSafetyUlps = 4;

// ---------------------------------------------------------------------------
// Build: q = clamp(rint(w / scale)), scale = max|w| * fl(1/127), residual_l2 = ||w - q * scale||_2
// rounded up by 8 ULPs (the arithmetic of native/src/native_lm_head.hip.cpp:53-115).
// One warp per row, 16-byte loads: lane l holds elements 256 g + 8 l + j (g, j in 0..7), writes its
// eight int8 results of a group with one 8-byte store.  The reference sums the squared residuals in
// FP64 as 256 partials (partial t = columns t, t + 256, ... in that order) folded by halving; a lane
// holds all eight columns of partials 8 l .. 8 l + 7, so the halvings of width 128 .. 8 are the lane
// butterfly of each partial and the last three are ((q0+q4)+(q2+q6))+((q1+q5)+(q3+q7)).
// ---------------------------------------------------------------------------
constexpr int kQuantizeWarps = 8;
__global__ void __launch_bounds__(kQuantizeWarps * 32)
lm_head_quantize_kernel(const __nv_bfloat16* __restrict__ source, int8_t* __restrict__ q_weight,
                        float* __restrict__ scales, float* __restrict__ residual_l2, int rows) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kQuantizeWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const size_t base = static_cast<size_t>(row) * kHidden;
  float v[64];
  float largest = 0.0f;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    unpack8(__ldg(reinterpret_cast<const uint4*>(source + base + 256 * g) + lane), v + 8 * g);
#pragma unroll
    for (int j = 0; j < 8; ++j) largest = fmaxf(largest, fabsf(v[8 * g + j]));
  }
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, s));
  const float scale = __fmul_rn(fmaxf(largest, 1.0e-12f), 1.0f / 127.0f);   // multiplication by the rounded reciprocal
  double partial[8] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float value = v[8 * g + j];
      const int quantized = static_cast<int>(fminf(127.0f, fmaxf(-127.0f, rintf(__fdiv_rn(value, scale)))));
      packed[j >> 2] |= (static_cast<uint32_t>(quantized) & 0xffu) << (8 * (j & 3));
      const double residual = static_cast<double>(__fsub_rn(value, __fmul_rn(static_cast<float>(quantized), scale)));
      partial[j] = __dadd_rn(partial[j], __dmul_rn(residual, residual));
    }
    *reinterpret_cast<uint2*>(q_weight + base + 256 * g + 8 * lane) = make_uint2(packed[0], packed[1]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) partial[j] = __dadd_rn(partial[j], __shfl_xor_sync(0xffffffffu, partial[j], s));
  }
  if (lane == 0) {
    const double total = __dadd_rn(__dadd_rn(__dadd_rn(partial[0], partial[4]), __dadd_rn(partial[2], partial[6])),
                                   __dadd_rn(__dadd_rn(partial[1], partial[5]), __dadd_rn(partial[3], partial[7])));
    float norm = static_cast<float>(sqrt(total));
    for (int step = 0; step < kResidualSafetyUlps; ++step) norm = nextafterf(norm, CUDART_INF_F);
    scales[row] = scale;
    residual_l2[row] = norm;
  }
}

// ---------------------------------------------------------------------------
// Scan: approximate[row] = scale[row] * sum_c q[row, c] * hidden[c], FP32.
// One warp per row at a time; lane l owns the 16-byte pieces l, l + 32, l + 64, l + 96 of the
// row (64 weights), multiplies them in ascending order into one accumulator, then the warp
// butterfly (16, 8, 4, 2, 1).  The lane's 64 hidden values stay in registers for all its rows.
// int8 -> FP32 without the conversion pipe: the byte, biased by 128, is placed in the mantissa
// of 2^23 and 2^23 + 128 is subtracted -- exact.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float byte_to_float(uint32_t biased_word, uint32_t selector) {
  return __fsub_rn(__uint_as_float(__byte_perm(biased_word, 0x4B000000u, selector)), 8388736.0f);
}

__device__ __forceinline__ float fma_word(uint32_t word, const float* x, float acc) {
  const uint32_t biased = word ^ 0x80808080u;
  acc = __fmaf_rn(byte_to_float(biased, 0x7540u), x[0], acc);
  acc = __fmaf_rn(byte_to_float(biased, 0x7541u), x[1], acc);
  acc = __fmaf_rn(byte_to_float(biased, 0x7542u), x[2], acc);
  acc = __fmaf_rn(byte_to_float(biased, 0x7543u), x[3], acc);
  return acc;
}

constexpr int kScanWarps = 4;

__global__ void __launch_bounds__(kScanWarps * 32)
lm_head_scan_kernel(const int8_t* __restrict__ q_weight, const float* __restrict__ scales,
                    const __nv_bfloat16* __restrict__ hidden, float* __restrict__ logits, int rows) {
  // the three short kernels after this one are placed while its last blocks drain (see pdl_enter)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * kScanWarps + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * kScanWarps;
  float x[64];
#pragma unroll
  for (int piece = 0; piece < 4; ++piece) {
    // 16 weights of piece (32 piece + lane): hidden elements 16 (32 piece + lane) .. + 15
    const uint4* src = reinterpret_cast<const uint4*>(hidden) + 2 * (32 * piece + lane);
    unpack8(__ldg(src), x + 16 * piece);
    unpack8(__ldg(src + 1), x + 16 * piece + 8);
  }
  // Two rows per trip, and the loads of the next trip are issued before the arithmetic of this one:
  // eight to sixteen 16-byte loads per lane stay in flight.
  auto load_pair = [&](int row, uint4* wa, uint4* wb) {
    const int row_b = row + warps_total;
    const uint4* qrow_a = reinterpret_cast<const uint4*>(q_weight + static_cast<size_t>(row) * kHidden) + lane;
    const uint4* qrow_b = reinterpret_cast<const uint4*>(q_weight + static_cast<size_t>(row_b < rows ? row_b : row) * kHidden) + lane;
#pragma unroll
    for (int piece = 0; piece < 4; ++piece) wa[piece] = __ldcs(qrow_a + 32 * piece);
#pragma unroll
    for (int piece = 0; piece < 4; ++piece) wb[piece] = __ldcs(qrow_b + 32 * piece);
  };
  uint4 wa[4], wb[4];
  if (warp_global < rows) load_pair(warp_global, wa, wb);
  for (int row = warp_global; row < rows; row += 2 * warps_total) {
    const int row_b = row + warps_total;
    const int next = row + 2 * warps_total;
    uint4 na[4], nb[4];
    if (next < rows) load_pair(next, na, nb);
    float acc_a = 0.0f, acc_b = 0.0f;
#pragma unroll
    for (int piece = 0; piece < 4; ++piece) {
      acc_a = fma_word(wa[piece].x, x + 16 * piece, acc_a);
      acc_a = fma_word(wa[piece].y, x + 16 * piece + 4, acc_a);
      acc_a = fma_word(wa[piece].z, x + 16 * piece + 8, acc_a);
      acc_a = fma_word(wa[piece].w, x + 16 * piece + 12, acc_a);
      acc_b = fma_word(wb[piece].x, x + 16 * piece, acc_b);
      acc_b = fma_word(wb[piece].y, x + 16 * piece + 4, acc_b);
      acc_b = fma_word(wb[piece].z, x + 16 * piece + 8, acc_b);
      acc_b = fma_word(wb[piece].w, x + 16 * piece + 12, acc_b);
    }
    acc_a = butterfly_sum(acc_a);
    acc_b = butterfly_sum(acc_b);
    if (lane == 0) {
      logits[row] = __fmul_rn(acc_a, scales[row]);
      if (row_b < rows) logits[row_b] = __fmul_rn(acc_b, scales[row_b]);
    }
    if (next < rows) {
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) { wa[piece] = na[piece]; wb[piece] = nb[piece]; }
    }
  }
}

// ||hidden||_2 in FP64 (thread-strided partials, pairwise tree), rounded to FP32 and up 4 ULPs.
// Every block of the bound kernel evaluates it for itself (2048 values) rather than waiting for
// a kernel of its own.
__device__ __forceinline__ float hidden_norm_in_block(const __nv_bfloat16* __restrict__ hidden, double* reduction) {
  const int t = threadIdx.x;
  double local = 0.0;
  for (int index = t; index < kHidden; index += kLmThreads) {
    const double value = static_cast<double>(__bfloat162float(hidden[index]));
    local = __dadd_rn(local, __dmul_rn(value, value));
  }
  reduction[t] = local;
  __syncthreads();
  for (int stride = kLmThreads / 2; stride != 0; stride >>= 1) {
    if (t < stride) reduction[t] = __dadd_rn(reduction[t], reduction[t + stride]);
    __syncthreads();
  }
  float norm = static_cast<float>(sqrt(reduction[0]));
  for (int step = 0; step < kHiddenSafetyUlps; ++step) norm = nextafterf(norm, CUDART_INF_F);
  return norm;
}

__device__ __forceinline__ float row_error(float residual, float hidden_l2) {
  return nextafterf(__fmul_rn(residual, hidden_l2), CUDART_INF_F);
}

// largest lower bound over all rows, per block; block 0 also publishes the hidden norm and empties
// the candidate list
__global__ void __launch_bounds__(kLmThreads)
lm_head_bound_kernel(const float* __restrict__ logits, const float* __restrict__ residual_l2,
                     const __nv_bfloat16* __restrict__ hidden, aima_moe_lm_head_result* wire,
                     float* __restrict__ partial, int rows) {
  __shared__ double norm_reduction[kLmThreads];
  __shared__ float reduction[kLmThreads];
  pdl_enter();
  const float hidden_l2 = hidden_norm_in_block(hidden, norm_reduction);
  float local_max = -CUDART_INF_F;
  for (int row = blockIdx.x * kLmThreads + threadIdx.x; row < rows; row += gridDim.x * kLmThreads) {
    const float lower = nextafterf(__fsub_rn(logits[row], row_error(residual_l2[row], hidden_l2)), -CUDART_INF_F);
    local_max = fmaxf(local_max, lower);
  }
  reduction[threadIdx.x] = local_max;
  __syncthreads();
  for (int stride = kLmThreads / 2; stride != 0; stride >>= 1) {
    if (threadIdx.x < stride) reduction[threadIdx.x] = fmaxf(reduction[threadIdx.x], reduction[threadIdx.x + stride]);
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    partial[blockIdx.x] = reduction[0];
    if (blockIdx.x == 0) {
      wire->hidden_l2 = hidden_l2;
      wire->candidate_count = 0;
      wire->overflow = 0;
    }
  }
}

// every row whose upper bound reaches the largest lower bound is a candidate; each block first
// reduces the 256 per-block maxima of the previous kernel
__global__ void __launch_bounds__(kLmThreads)
lm_head_collect_kernel(const float* __restrict__ logits, const float* __restrict__ residual_l2,
                       const float* __restrict__ partial, aima_moe_lm_head_result* wire,
                       uint32_t* __restrict__ candidate_ids, int rows) {
  static_assert(kLmThreads == kLmBoundBlocks, "one thread per partial maximum");
  __shared__ float reduction[kLmBoundBlocks];
  pdl_enter();
  reduction[threadIdx.x] = partial[threadIdx.x];
  __syncthreads();
  for (int stride = kLmBoundBlocks / 2; stride != 0; stride >>= 1) {
    if (threadIdx.x < stride) reduction[threadIdx.x] = fmaxf(reduction[threadIdx.x], reduction[threadIdx.x + stride]);
    __syncthreads();
  }
  const float maximum_lower_bound = reduction[0];
  if (blockIdx.x == 0 && threadIdx.x == 0) wire->maximum_lower_bound = maximum_lower_bound;
  const int row = blockIdx.x * kLmThreads + threadIdx.x;
  if (row >= rows) return;
  const float upper = nextafterf(__fadd_rn(logits[row], row_error(residual_l2[row], wire->hidden_l2)), CUDART_INF_F);
  if (upper < maximum_lower_bound) return;
  const uint32_t slot = atomicAdd(&wire->candidate_count, 1u);
  if (slot < AIMA_MOE_LM_HEAD_CANDIDATES) candidate_ids[slot] = static_cast<uint32_t>(row);
  else wire->overflow = 1;
}

__device__ __forceinline__ bool better(float value, uint32_t index, float current, uint32_t current_index) {
  return value > current || (value == current && index < current_index);
}

// One block: the exact BF16 logit of every candidate straight from the raw matrix (no gathered
// copy) -- the canonical warp dot, rounded to BF16 like the reference's N = 1 GEMV provider -- then
// the exact top-1 over them.  The exact logits replace the approximate ones in `logits`.
constexpr int kExactWarps = 32;
__global__ void __launch_bounds__(kExactWarps * 32)
lm_head_exact_kernel(const __nv_bfloat16* __restrict__ weight, const __nv_bfloat16* __restrict__ hidden,
                     aima_moe_lm_head_result* wire, const uint32_t* __restrict__ candidate_ids,
                     float* __restrict__ logits) {
  __shared__ float values[kExactWarps];
  __shared__ uint32_t indices[kExactWarps];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  pdl_enter();
  const uint32_t count = min(wire->candidate_count, static_cast<uint32_t>(AIMA_MOE_LM_HEAD_CANDIDATES));
  const uint4* xrow = reinterpret_cast<const uint4*>(hidden) + lane;
  float local_value = -CUDART_INF_F;
  uint32_t local_index = 0;
  for (uint32_t candidate = warp; candidate < count; candidate += kExactWarps) {
    const uint32_t token = candidate_ids[candidate];
    const uint4* wrow = reinterpret_cast<const uint4*>(weight + static_cast<size_t>(token) * kHidden) + lane;
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < kHidden / 256; ++i) {
      float xf[8];
      unpack8(__ldg(xrow + i * 32), xf);
      acc = fma8(xf, __ldg(wrow + i * 32), acc);
    }
    acc = butterfly_sum(acc);
    const float value = round_bf16(acc);
    if (lane == 0) logits[token] = value;
    if (better(value, token, local_value, local_index)) { local_value = value; local_index = token; }
  }
  if (lane == 0) { values[warp] = local_value; indices[warp] = local_index; }
  __syncthreads();
  if (warp == 0) {
    float value = values[lane];
    uint32_t index = indices[lane];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other_value = __shfl_xor_sync(0xffffffffu, value, offset);
      const uint32_t other_index = __shfl_xor_sync(0xffffffffu, index, offset);
      if (better(other_value, other_index, value, index)) { value = other_value; index = other_index; }
    }
    if (lane == 0) {
      wire->exact_top1_logit = value;
      wire->exact_top1_token_id = index;
    }
  }
}

}  // namespace

cudaError_t lm_head_quantize(const void* weight, int rows, int8_t* q_weight, float* scales, float* residual_l2,
                             cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  lm_head_quantize_kernel<<<(rows + kQuantizeWarps - 1) / kQuantizeWarps, kQuantizeWarps * 32, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(weight), q_weight, scales, residual_l2, rows);
  return cudaGetLastError();
}

cudaError_t lm_head_certify(const LmHeadBuffers& b, const void* weight, const void* hidden, float* logits,
                            int rows, int sm_count, cudaStream_t stream, int* launches) {
  const __nv_bfloat16* h = static_cast<const __nv_bfloat16*>(hidden);
  lm_head_scan_kernel<<<sm_count * 16, kScanWarps * 32, 0, stream>>>(b.q_weight, b.scales, h, logits, rows);
  cudaError_t code = cudaGetLastError();
  const PdlScope pdl_scope(true);
  if (code == cudaSuccess)
    code = launch_pdl(lm_head_bound_kernel, dim3(kLmBoundBlocks), dim3(kLmThreads), 0, stream,
                      static_cast<const float*>(logits), static_cast<const float*>(b.residual_l2), h, b.wire, b.partial, rows);
  if (code == cudaSuccess)
    code = launch_pdl(lm_head_collect_kernel, dim3((rows + kLmThreads - 1) / kLmThreads), dim3(kLmThreads), 0, stream,
                      static_cast<const float*>(logits), static_cast<const float*>(b.residual_l2),
                      static_cast<const float*>(b.partial), b.wire, b.candidate_ids, rows);
  if (code == cudaSuccess)
    code = launch_pdl(lm_head_exact_kernel, dim3(1), dim3(kExactWarps * 32), 0, stream,
                      static_cast<const __nv_bfloat16*>(weight), h, b.wire, b.candidate_ids, logits);
  *launches = 4;
  return code;
}

}  // namespace aima
