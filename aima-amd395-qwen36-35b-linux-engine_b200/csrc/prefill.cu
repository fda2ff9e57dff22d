// Prefill MoE half-layer on the GPU: router + top-8, dispatch plan, gather,
// grouped expert products, shared expert, weighted combine.
//
// Stage list and rounding points follow the reference orchestration
// (native/src/native_moe_prefill.hip.cpp:790-893):
//   router GEMM -> BF16 logits -> router_topk8_softmax_256_kernel (:234-323)
//   moe_align_block32_256_kernel (:325-382)            -> here: a deterministic
//       counting sort into a per-expert offset table (no padding rows)
//   fused_moe_kernel gate_up -> expert_silu_multiply_kernel (:384-402)
//   fused_moe_kernel down (x routing weight)           -> moe_sum8_kernel (:404-431)
//   shared expert (:210-232, 790-826), bf16_add_pair_kernel
//   (native/src/native_pointwise.hip.cpp:94-107)
#include "prefill.cuh"

#include "grouped_gemm.cuh"

#include <cstdio>
#include <math_constants.h>

namespace aima {
namespace {

// Monotone map FP32 -> uint32 (larger float <=> larger key), for redux-based maxima.
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// 8th largest of the 256 values a warp holds (8 per lane), counting repeats.
__device__ __forceinline__ float warp_eighth_largest(const float* v, int lane) {
  uint32_t k[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) k[q] = order_key(v[q]);
  uint32_t best = 0;
#pragma unroll
  for (int r = 0; r < kTopK; ++r) {
    uint32_t local = k[0];
#pragma unroll
    for (int q = 1; q < 8; ++q) local = max(local, k[q]);
    best = __reduce_max_sync(0xffffffffu, local);
    const unsigned owners = __ballot_sync(0xffffffffu, local == best);
    if (lane == __ffs(owners) - 1) {
      bool removed = false;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (!removed && k[q] == best) { k[q] = 0u; removed = true; }
      }
    }
  }
  return key_value(best);
}

// The reference's prefill selection on the final (BF16-rounded) logits of one
// token held as v[q] = logit of expert 32 q + lane: threshold, gather in expert
// order, fixed bitonic network, softmax; lanes 0..7 write slot `lane`.
__device__ __forceinline__ int route_token(const float* v, int lane, float* sel_v, int* sel_i,
                                            size_t token, int32_t* __restrict__ ids,
                                            float* __restrict__ scores, float* __restrict__ weights,
                                            __nv_bfloat16* __restrict__ dbg_weights) {
  const float threshold = warp_eighth_largest(v, lane);
  const unsigned lt_mask = (1u << lane) - 1u;
  int held = 0;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const bool take = v[q] > threshold;
    const unsigned m = __ballot_sync(0xffffffffu, take);
    if (take) {
      const int pos = held + __popc(m & lt_mask);
      sel_v[pos] = v[q];
      sel_i[pos] = 32 * q + lane;
    }
    held += __popc(m);
  }
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const bool take = v[q] == threshold;
    const unsigned m = __ballot_sync(0xffffffffu, take);
    if (take) {
      const int pos = held + __popc(m & lt_mask);
      if (pos < kTopK) {
        sel_v[pos] = v[q];
        sel_i[pos] = 32 * q + lane;
      }
    }
    held += __popc(m);
  }
  __syncwarp();
  float sv[kTopK];
  int si[kTopK];
#pragma unroll
  for (int r = 0; r < kTopK; ++r) { sv[r] = sel_v[r]; si[r] = sel_i[r]; }
  __syncwarp();
  // fixed 8-wide bitonic network; a pair is exchanged when
  // (value[left] > value[right]) equals the "ascending" flag of the left index
#pragma unroll
  for (int width = 2; width <= kTopK; width *= 2) {
#pragma unroll
    for (int stride = width / 2; stride > 0; stride /= 2) {
#pragma unroll
      for (int left = 0; left < kTopK; ++left) {
        const int right = left ^ stride;
        if (right > left) {
          const bool ascending = (left & width) != 0;
          if ((sv[left] > sv[right]) == ascending) {
            const float tv = sv[left]; sv[left] = sv[right]; sv[right] = tv;
            const int ti = si[left]; si[left] = si[right]; si[right] = ti;
          }
        }
      }
    }
  }
  float ex[kTopK];
  float denom = 0.0f;
#pragma unroll
  for (int r = 0; r < kTopK; ++r) {
    ex[r] = det_expf(__fsub_rn(sv[r], sv[0]));
    denom = __fadd_rn(denom, ex[r]);
  }
#pragma unroll
  for (int r = 0; r < kTopK; ++r) {
    if (lane == r) {
      const size_t o = token * kTopK + r;
      const uint16_t wb = float_to_bf16_bits(__fdiv_rn(ex[r], denom));
      ids[o] = si[r];
      scores[o] = sv[r];
      weights[o] = bf16_bits_to_float(wb);
      if (dbg_weights != nullptr) reinterpret_cast<uint16_t*>(dbg_weights)[o] = wb;
    }
  }
  int selected = -1;      // lane r < 8 returns the expert of slot r
#pragma unroll
  for (int r = 0; r < kTopK; ++r) {
    if (lane == r) selected = si[r];
  }
  return selected;
}

// logit transform shared by both router kernels: optional harness hooks, then
// the BF16 rounding the reference's router GEMM applies
__device__ __forceinline__ float finish_logit(float x, float bias, int quant_eighths) {
  x = __fadd_rn(x, bias);
  if (quant_eighths) x = __fmul_rn(rintf(__fmul_rn(x, 8.0f)), 0.125f);
  return round_bf16(x);
}

// ---------------------------------------------------------------------------
// Router: canonical FP32 logits of all 256 experts (+ the shared-expert gate
// row), BF16 rounding, the reference's selection rule and softmax.
// One warp per token, 16 tokens per block; router rows are staged through
// shared memory 32 at a time.
// ---------------------------------------------------------------------------
constexpr int kRouterWarps = 16;
constexpr int kRouterChunkRows = 32;
constexpr int kRouterSmemBytes = kRouterChunkRows * kHidden * 2 + kRouterWarps * 8 * 8;

__global__ void __launch_bounds__(kRouterWarps * 32, 1)
prefill_router_kernel(const __nv_bfloat16* __restrict__ h2,
                      const __nv_bfloat16* __restrict__ router,
                      const __nv_bfloat16* __restrict__ shared_gate,
                      const float* __restrict__ bias, int quant_eighths, int tokens,
                      int32_t* __restrict__ ids, float* __restrict__ scores,
                      float* __restrict__ weights, float* __restrict__ shared_sigmoid,
                      float* __restrict__ dbg_logits, __nv_bfloat16* __restrict__ dbg_weights) {
  extern __shared__ __align__(16) uint8_t smem[];
  uint4* rows_s = reinterpret_cast<uint4*>(smem);
  float* sel_v_s = reinterpret_cast<float*>(smem + kRouterChunkRows * kHidden * 2);
  int* sel_i_s = reinterpret_cast<int*>(sel_v_s + kRouterWarps * 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * kRouterWarps + warp;
  const bool valid = token < tokens;

  float xr[64];
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (valid) v = *(reinterpret_cast<const uint4*>(h2 + static_cast<size_t>(token) * kHidden) + g * 32 + lane);
    unpack8(v, xr + 8 * g);
  }

  float v[8];   // lane l holds the logit of expert 32 q + l in v[q]
  float gate_dot = 0.0f;
#pragma unroll
  for (int chunk = 0; chunk < 9; ++chunk) {
    const int n_rows = (chunk < 8) ? kRouterChunkRows : 1;
    const __nv_bfloat16* src = (chunk < 8) ? router + static_cast<size_t>(chunk) * kRouterChunkRows * kHidden
                                           : shared_gate;
    __syncthreads();
    for (int i = threadIdx.x; i < n_rows * (kHidden / 8); i += blockDim.x) {
      rows_s[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
    }
    __syncthreads();
    if (chunk < 8) {
      float mine = 0.0f;
      for (int r = 0; r < kRouterChunkRows; r += 2) {
        const uint4* r0 = rows_s + r * (kHidden / 8) + lane;
        const uint4* r1 = r0 + (kHidden / 8);
        float a = 0.0f, b = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          a = fma8(xr + 8 * i, r0[i * 32], a);
          b = fma8(xr + 8 * i, r1[i * 32], b);
        }
        a = butterfly_sum(a);
        b = butterfly_sum(b);
        if (lane == r) mine = a;
        if (lane == r + 1) mine = b;
      }
      v[chunk] = mine;
    } else {
      const uint4* r0 = rows_s + lane;
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) a = fma8(xr + 8 * i, r0[i * 32], a);
      gate_dot = butterfly_sum(a);
    }
  }
  if (!valid) return;

  // harness hooks, then the BF16 rounding the reference's router GEMM applies
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    v[q] = finish_logit(v[q], bias != nullptr ? bias[32 * q + lane] : 0.0f, quant_eighths);
    if (dbg_logits != nullptr) dbg_logits[static_cast<size_t>(token) * kExperts + 32 * q + lane] = v[q];
  }
  route_token(v, lane, sel_v_s + warp * 8, sel_i_s + warp * 8, static_cast<size_t>(token), ids, scores,
              weights, dbg_weights);
  if (lane == 0) {
    shared_sigmoid[token] = round_bf16(det_sigmoid(round_bf16(gate_dot)));
  }
}

// ---------------------------------------------------------------------------
// Certified router.  All 256 logits come from the tensor cores first (FP32,
// unknown accumulation order, `approx`).  Their distance to the canonical value
// is bounded by kappa * |x|_2 * |w_e|_2 (Cauchy-Schwarz on the FP32 rounding
// error of a 2048-term sum, in the spirit of the reference's certified LM head,
// native/src/native_lm_head_certificate.hip.cpp:33-39).  Only experts whose
// upper bound reaches the lower bound of the 8th-largest value can be selected;
// those few are recomputed with the canonical dot and the reference's rule runs
// on them alone, so ids, scores and weights stay bit-exact.
//
// The bound is a statement about hardware whose accumulation order is not
// published, so the kernel checks it where it can: every candidate has both
// values, and if one lies further from its tensor-core value than the bound
// allows, the whole token is recomputed with the canonical dot (all 256
// experts) and counted.  With audit_stride > 0 every audit_stride-th token is
// recomputed in full as well and its ids compared with the certified ones.
// One warp per token.
// ---------------------------------------------------------------------------
constexpr int kCertWarps = 8;
constexpr float kCertKappa = 6.103515625e-05f;   // 2^-14, ~4x the summed worst-case rounding terms

// canonical 8-element step of the warp dot with BOTH operands still packed (same FMA order as fma8)
__device__ __forceinline__ float fma8_packed(const uint4& x, const uint4& w, float acc) {
  acc = __fmaf_rn(bf16_lo(x.x), bf16_lo(w.x), acc);
  acc = __fmaf_rn(bf16_hi(x.x), bf16_hi(w.x), acc);
  acc = __fmaf_rn(bf16_lo(x.y), bf16_lo(w.y), acc);
  acc = __fmaf_rn(bf16_hi(x.y), bf16_hi(w.y), acc);
  acc = __fmaf_rn(bf16_lo(x.z), bf16_lo(w.z), acc);
  acc = __fmaf_rn(bf16_hi(x.z), bf16_hi(w.z), acc);
  acc = __fmaf_rn(bf16_lo(x.w), bf16_lo(w.w), acc);
  acc = __fmaf_rn(bf16_hi(x.w), bf16_hi(w.w), acc);
  return acc;
}

// The token's row stays packed in registers, and the candidates are recomputed two at a time: the
// kernel is bound by the latency of the candidates' router rows coming from L2, so two rows are
// requested before either is used.
__global__ void __launch_bounds__(kCertWarps * 32, 2)
prefill_router_certified_kernel(const __nv_bfloat16* __restrict__ h2,
                                const __nv_bfloat16* __restrict__ router,
                                const __nv_bfloat16* __restrict__ shared_gate,
                                const float* __restrict__ approx,
                                const float* __restrict__ row_norms,
                                const float* __restrict__ bias, int quant_eighths, int tokens,
                                int32_t* __restrict__ ids, float* __restrict__ scores,
                                float* __restrict__ weights, float* __restrict__ shared_sigmoid,
                                __nv_bfloat16* __restrict__ dbg_weights, int32_t* __restrict__ stats,
                                int audit_stride) {
  __shared__ float sel_v_s[kCertWarps * 8];
  __shared__ int sel_i_s[kCertWarps * 8];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * kCertWarps + warp;
  pdl_enter();
  if (token >= tokens) return;

  uint4 xp[8];
  float sumsq = 0.0f;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    xp[g] = *(reinterpret_cast<const uint4*>(h2 + static_cast<size_t>(token) * kHidden) + g * 32 + lane);
    float x8[8];
    unpack8(xp[g], x8);
#pragma unroll
    for (int j = 0; j < 8; ++j) sumsq = fmaf(x8[j], x8[j], sumsq);
  }
  sumsq = butterfly_sum(sumsq);
  const float x_norm = sqrtf(sumsq) * 1.0001f;

  float upper[8], lower[8], b[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int e = 32 * q + lane;
    b[q] = bias != nullptr ? bias[e] : 0.0f;
    const float a = approx[static_cast<size_t>(token) * kExperts + e];
    const float delta = kCertKappa * x_norm * row_norms[e] + 9.5367431640625e-07f * fabsf(a + b[q]);
    upper[q] = finish_logit(a + delta, b[q], quant_eighths);
    lower[q] = finish_logit(a - delta, b[q], quant_eighths);
  }
  const float floor_value = warp_eighth_largest(lower, lane);

  // lane q (q < 8) keeps the candidate mask of experts 32 q .. 32 q + 31; the warp walks all masks
  // and takes two candidates per trip
  unsigned my_mask = 0u;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const unsigned m = __ballot_sync(0xffffffffu, upper[q] >= floor_value);
    if (lane == q) my_mask = m;
  }
  float v[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) v[q] = -CUDART_INF_F;
  int recomputed = 0;
  int group = 0;
  unsigned pending = __shfl_sync(0xffffffffu, my_mask, 0);
  auto pop = [&]() -> int {
    while (pending == 0u) {
      if (++group >= 8) return -1;
      pending = __shfl_sync(0xffffffffu, my_mask, group);
    }
    const int owner = __ffs(pending) - 1;
    pending &= pending - 1u;
    return 32 * group + owner;
  };
  // canonical logits of two experts at once (e1 < 0: only e0); the owner lanes file them in v
  auto exact_pair = [&](int e0, int e1, float& acc0, float& acc1) {
    const uint4* row0 = reinterpret_cast<const uint4*>(router + static_cast<size_t>(e0) * kHidden) + lane;
    const uint4* row1 = reinterpret_cast<const uint4*>(router + static_cast<size_t>(e1 >= 0 ? e1 : e0) * kHidden) + lane;
    uint4 w0[8], w1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w0[i] = __ldg(row0 + i * 32);
#pragma unroll
    for (int i = 0; i < 8; ++i) w1[i] = __ldg(row1 + i * 32);
    acc0 = 0.0f;
    acc1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      acc0 = fma8_packed(xp[i], w0[i], acc0);
      acc1 = fma8_packed(xp[i], w1[i], acc1);
    }
    acc0 = butterfly_sum(acc0);
    acc1 = butterfly_sum(acc1);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (e0 == 32 * q + lane) v[q] = finish_logit(acc0, b[q], quant_eighths);
      if (e1 == 32 * q + lane) v[q] = finish_logit(acc1, b[q], quant_eighths);
    }
  };
  // is the canonical value further from the tensor-core value than the bound the filter relied on?
  auto outside_bound = [&](float exact, int e) -> bool {
    const float a = approx[static_cast<size_t>(token) * kExperts + e];
    const float be = bias != nullptr ? bias[e] : 0.0f;
    const float delta = kCertKappa * x_norm * row_norms[e] + 9.5367431640625e-07f * fabsf(a + be);
    return fabsf(exact - a) > delta;
  };
  bool violated = false;
  while (true) {
    const int e0 = pop();
    if (e0 < 0) break;
    const int e1 = pop();
    float acc0, acc1;
    exact_pair(e0, e1, acc0, acc1);
    if ((e0 & 31) == lane) violated = violated || outside_bound(acc0, e0);
    if (e1 >= 0 && (e1 & 31) == lane) violated = violated || outside_bound(acc1, e1);
    recomputed += e1 >= 0 ? 2 : 1;
  }
  violated = __any_sync(0xffffffffu, violated);
  if (violated) {
    // the premise of the filter failed for this token: take nothing from it
    for (int e = 0; e < kExperts; e += 2) {
      float acc0, acc1;
      exact_pair(e, e + 1, acc0, acc1);
    }
  }
  const int certified_id = route_token(v, lane, sel_v_s + warp * 8, sel_i_s + warp * 8, static_cast<size_t>(token),
                                       ids, scores, weights, dbg_weights);
  bool audited = false, audit_mismatch = false;
  if (audit_stride > 0 && token % audit_stride == 0 && !violated) {
    for (int e = 0; e < kExperts; e += 2) {
      float acc0, acc1;
      exact_pair(e, e + 1, acc0, acc1);
    }
    const int exact_id = route_token(v, lane, sel_v_s + warp * 8, sel_i_s + warp * 8, static_cast<size_t>(token),
                                     ids, scores, weights, dbg_weights);
    audited = true;
    audit_mismatch = __any_sync(0xffffffffu, lane < kTopK && exact_id != certified_id);
  }
  {
    const uint4* row = reinterpret_cast<const uint4*>(shared_gate) + lane;
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fma8_packed(xp[i], __ldg(row + i * 32), acc);
    acc = butterfly_sum(acc);
    if (lane == 0) {
      shared_sigmoid[token] = round_bf16(det_sigmoid(round_bf16(acc)));
      if (stats != nullptr) {
        atomicAdd(stats, recomputed);
        atomicAdd(stats + 1, 1);
        if (violated) atomicAdd(stats + 2, 1);
        if (audited) atomicAdd(stats + 3, 1);
        if (audit_mismatch) atomicAdd(stats + 4, 1);
      }
    }
  }
}

// Euclidean norms of the 256 router rows, rounded up a little; one warp per row.
__global__ void __launch_bounds__(256)
router_row_norms_kernel(const __nv_bfloat16* __restrict__ router, float* __restrict__ norms) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= kExperts) return;
  const uint4* src = reinterpret_cast<const uint4*>(router + static_cast<size_t>(row) * kHidden) + lane;
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float w[8];
    unpack8(__ldg(src + i * 32), w);
#pragma unroll
    for (int j = 0; j < 8; ++j) sum = fmaf(w[j], w[j], sum);
  }
  sum = butterfly_sum(sum);
  if (lane == 0) norms[row] = sqrtf(sum) * 1.0001f;
}

// ---------------------------------------------------------------------------
// Dispatch plan: stable counting sort of the 8T routed rows by expert.
// A "unit" is the 256 consecutive flat rows one warp owns.
// ---------------------------------------------------------------------------
constexpr int kPlanWarps = 8;

__global__ void __launch_bounds__(kPlanWarps * 32)
plan_count_kernel(const int32_t* __restrict__ ids, int routed_rows, int expert_lo, int expert_hi,
                  int32_t* __restrict__ unit_counts) {
  __shared__ int cnt[kPlanWarps][kExperts];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int e = lane; e < kExperts; e += 32) cnt[warp][e] = 0;
  __syncwarp();
  pdl_enter();
  const int unit = blockIdx.x * kPlanWarps + warp;
  const int row0 = unit * kPlanRowsPerWarp;
  if (row0 >= routed_rows) return;
  for (int round = 0; round < kPlanRowsPerWarp / 32; ++round) {
    const int row = row0 + round * 32 + lane;
    // rows routed to experts held by another GPU are not part of this GPU's plan
    const int e = row < routed_rows ? ids[row] : -1;
    const bool valid = e >= expert_lo && e < expert_hi;
    const unsigned active = __ballot_sync(0xffffffffu, valid);
    if (valid) {
      const unsigned same = __match_any_sync(active, e);
      if ((same & ((1u << lane) - 1u)) == 0u) cnt[warp][e] += __popc(same);
    }
    __syncwarp();
  }
  for (int e = lane; e < kExperts; e += 32) {
    unit_counts[static_cast<size_t>(unit) * kExperts + e] = cnt[warp][e];
  }
}

// One warp per expert: exclusive prefix of that expert's counts over the units (in place) and the
// expert's total.  Grid = 256 / kPlanWarps blocks.
__global__ void __launch_bounds__(kPlanWarps * 32)
plan_scan_kernel(int32_t* __restrict__ unit_counts, int units, int32_t* __restrict__ expert_counts) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * kPlanWarps + (threadIdx.x >> 5);
  int running = 0;
  for (int u0 = 0; u0 < units; u0 += 32) {
    const int u = u0 + lane;
    const size_t index = static_cast<size_t>(u) * kExperts + e;
    const int c = u < units ? unit_counts[index] : 0;
    int inclusive = c;
#pragma unroll
    for (int d = 1; d < 32; d *= 2) {
      const int up = __shfl_up_sync(0xffffffffu, inclusive, d);
      if (lane >= d) inclusive += up;
    }
    if (u < units) unit_counts[index] = running + inclusive - c;
    running += __shfl_sync(0xffffffffu, inclusive, 31);
  }
  if (lane == 0) expert_counts[e] = running;
}

// Exclusive offsets of the 256 experts from their counts, in shared memory (all 256 threads of a
// block take part); thread 0 .. 255 returns with offsets[0 .. 256] and tile_base[0 .. 256] filled.
__device__ __forceinline__ int expert_offsets_in_block(const int32_t* __restrict__ expert_counts, int tile_cap,
                                                       int* offsets, int* tile_base, int* warp_sums) {
  const int e = threadIdx.x;
  const int lane = e & 31, warp = e >> 5;
  const int count = expert_counts[e];
  int v0 = count, v1 = (count + tile_cap - 1) / tile_cap, v2 = (count + 31) / 32 * 32;
  const int mine0 = v0, mine1 = v1;
#pragma unroll
  for (int d = 1; d < 32; d *= 2) {
    const int a0 = __shfl_up_sync(0xffffffffu, v0, d);
    const int a1 = __shfl_up_sync(0xffffffffu, v1, d);
    const int a2 = __shfl_up_sync(0xffffffffu, v2, d);
    if (lane >= d) { v0 += a0; v1 += a1; v2 += a2; }
  }
  if (lane == 31) { warp_sums[warp] = v0; warp_sums[8 + warp] = v1; warp_sums[16 + warp] = v2; }
  __syncthreads();
  int b0 = 0, b1 = 0, padded = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    if (w < warp) { b0 += warp_sums[w]; b1 += warp_sums[8 + w]; }
    padded += warp_sums[16 + w];
  }
  offsets[e] = b0 + v0 - mine0;
  tile_base[e] = b1 + v1 - mine1;
  if (e == kExperts - 1) { offsets[kExperts] = b0 + v0; tile_base[kExperts] = b1 + v1; }
  __syncthreads();
  return padded;
}

// Stable scatter.  Every block first derives the expert offsets from the counts; block 0 also
// publishes them together with the tile list and the reference's block-32 padded row count.
__global__ void __launch_bounds__(kPlanWarps * 32)
plan_scatter_kernel(const int32_t* __restrict__ ids, int routed_rows, int expert_lo, int expert_hi,
                    const int32_t* __restrict__ unit_prefix,
                    const int32_t* __restrict__ expert_counts,
                    int32_t* __restrict__ expert_offsets,
                    int32_t* __restrict__ tile_expert, int32_t* __restrict__ tile_row0,
                    int32_t* __restrict__ tile_rows, int32_t* __restrict__ tile_count,
                    int32_t* __restrict__ padded_rows,
                    int32_t* __restrict__ sorted_rows, int32_t* __restrict__ row_position, int tile_cap) {
  static_assert(kPlanWarps * 32 == kExperts, "one thread per expert in the prologue");
  pdl_enter();
  __shared__ int next[kPlanWarps][kExperts];
  __shared__ int offsets[kExperts + 1];
  __shared__ int tile_base[kExperts + 1];
  __shared__ int warp_sums[24];
  const int padded = expert_offsets_in_block(expert_counts, tile_cap, offsets, tile_base, warp_sums);
  if (blockIdx.x == 0) {
    const int e = threadIdx.x;
    const int count = offsets[e + 1] - offsets[e];
    expert_offsets[e] = offsets[e];
    if (e == 0) {
      expert_offsets[kExperts] = offsets[kExperts];
      *tile_count = tile_base[kExperts];
      *padded_rows = padded;
    }
    const int n_tiles = tile_base[e + 1] - tile_base[e];
    for (int t = 0; t < n_tiles; ++t) {
      const int index = tile_base[e] + t;
      tile_expert[index] = e;
      tile_row0[index] = offsets[e] + t * tile_cap;
      tile_rows[index] = min(tile_cap, count - t * tile_cap);
    }
  }
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * kPlanWarps + warp;
  const int row0 = unit * kPlanRowsPerWarp;
  if (row0 >= routed_rows) return;
  for (int e = lane; e < kExperts; e += 32) {
    next[warp][e] = offsets[e] + unit_prefix[static_cast<size_t>(unit) * kExperts + e];
  }
  __syncwarp();
  for (int round = 0; round < kPlanRowsPerWarp / 32; ++round) {
    const int row = row0 + round * 32 + lane;
    const int e = row < routed_rows ? ids[row] : -1;
    const bool valid = e >= expert_lo && e < expert_hi;
    const unsigned active = __ballot_sync(0xffffffffu, valid);
    if (valid) {
      const unsigned same = __match_any_sync(active, e);
      const int rank = __popc(same & ((1u << lane) - 1u));
      const int pos = next[warp][e] + rank;
      sorted_rows[pos] = row;
      row_position[row] = pos;
      __syncwarp(active);
      if (rank == 0) next[warp][e] += __popc(same);
    }
    __syncwarp();
  }
}

// Enqueues the dispatch plan for `rows` routed rows whose expert ids are `ids`.
// tile_cap: rows per tile of the plan -- 128 for the one-SM product kernels, 256 for the two-SM form
cudaError_t launch_plan(PrefillWorkspace* ws, const int32_t* ids, int rows, int expert_lo, int expert_hi,
                        cudaStream_t stream, int* launches, int tile_cap = kTileRows) {
  const int units = (rows + kPlanRowsPerWarp - 1) / kPlanRowsPerWarp;
  const int plan_blocks = (units + kPlanWarps - 1) / kPlanWarps;
  cudaError_t code = launch_pdl(plan_count_kernel, dim3(plan_blocks), dim3(kPlanWarps * 32), 0, stream, ids, rows,
                                expert_lo, expert_hi, ws->unit_counts);
  if (code == cudaSuccess)
    code = launch_pdl(plan_scan_kernel, dim3(kExperts / kPlanWarps), dim3(kPlanWarps * 32), 0, stream,
                      ws->unit_counts, units, ws->expert_counts);
  if (code == cudaSuccess)
    code = launch_pdl(plan_scatter_kernel, dim3(plan_blocks), dim3(kPlanWarps * 32), 0, stream, ids, rows,
                      expert_lo, expert_hi, ws->unit_counts, ws->expert_counts, ws->expert_offsets,
                      ws->tile_expert, ws->tile_row0, ws->tile_rows, ws->tile_count, ws->padded_rows,
                      ws->sorted_rows, ws->row_position, tile_cap);
  *launches += 3;
  return code;
}

// ---------------------------------------------------------------------------
// Gather of h2 rows into expert order; one warp per routed row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ h2, const int32_t* __restrict__ sorted_rows,
                   int routed_rows, __nv_bfloat16* __restrict__ gathered) {
  const int lane = threadIdx.x & 31;
  const int pos = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (pos >= routed_rows) return;
  const int token = sorted_rows[pos] >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(h2 + static_cast<size_t>(token) * kHidden);
  uint4* dst = reinterpret_cast<uint4*>(gathered + static_cast<size_t>(pos) * kHidden);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i * 32 + lane] = __ldg(src + i * 32 + lane);
}

// ---------------------------------------------------------------------------
// Combine: routed = bf16((((r0+r4)+(r1+r5))+(r2+r6))+(r3+r7)) over the eight
// weighted expert outputs of a token, combined = bf16(routed + shared),
// out = bf16(residual + combined).  One block of 256 threads per token.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
combine_kernel(const __nv_bfloat16* __restrict__ expert_down,
               const int32_t* __restrict__ row_position,
               const __nv_bfloat16* __restrict__ shared_scaled,
               const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
               __nv_bfloat16* __restrict__ dbg_routed,
               const __nv_bfloat16* __restrict__ next_norm_weight,
               __nv_bfloat16* __restrict__ next_norm_out, float eps) {
  __shared__ float group_sums[8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // next layer's router product may set itself up
  const int token = blockIdx.x;
  const int t = threadIdx.x;
  float slot[kTopK][8];
#pragma unroll
  for (int s = 0; s < kTopK; ++s) {
    const int pos = row_position != nullptr ? row_position[token * kTopK + s] : token * kTopK + s;
    unpack8(__ldg(reinterpret_cast<const uint4*>(expert_down + static_cast<size_t>(pos) * kHidden) + t),
            slot[s]);
  }
  float sh[8], rs[8];
  const size_t base = static_cast<size_t>(token) * kHidden;
  unpack8(__ldg(reinterpret_cast<const uint4*>(shared_scaled + base) + t), sh);
  unpack8(__ldg(reinterpret_cast<const uint4*>(residual + base) + t), rs);
  uint32_t packed[4], packed_routed[4];
  float o8[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float s04 = __fadd_rn(slot[0][j], slot[4][j]);
    const float s15 = __fadd_rn(slot[1][j], slot[5][j]);
    const float s26 = __fadd_rn(slot[2][j], slot[6][j]);
    const float s37 = __fadd_rn(slot[3][j], slot[7][j]);
    float sum = __fadd_rn(s04, s15);
    sum = __fadd_rn(sum, s26);
    sum = __fadd_rn(sum, s37);
    const uint16_t routed_bits = float_to_bf16_bits(sum);
    const float combined = round_bf16(__fadd_rn(bf16_bits_to_float(routed_bits), sh[j]));
    const uint16_t o = float_to_bf16_bits(__fadd_rn(rs[j], combined));
    o8[j] = bf16_bits_to_float(o);
    if (j & 1) {
      packed[j / 2] |= static_cast<uint32_t>(o) << 16;
      packed_routed[j / 2] |= static_cast<uint32_t>(routed_bits) << 16;
    } else {
      packed[j / 2] = o;
      packed_routed[j / 2] = routed_bits;
    }
  }
  reinterpret_cast<uint4*>(out + base)[t] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  if (dbg_routed != nullptr) {
    reinterpret_cast<uint4*>(dbg_routed + base)[t] =
        make_uint4(packed_routed[0], packed_routed[1], packed_routed[2], packed_routed[3]);
  }
  // Optional exit: RMSNorm of the row just produced (the next layer's input norm).  Sum of squares in
  // the order of the reference kernel (native/src/native_pointwise.hip.cpp:109-142): partial p of 256
  // adds elements p, p + 256, ... in that order, the partials fold by halving.  Thread t holds elements
  // 8 t .. 8 t + 7, so the squares go through shared memory once and thread p picks up its eight.
  if (next_norm_out != nullptr) {
    __shared__ float squares[kHidden];
    __shared__ float partial[256];
#pragma unroll
    for (int j = 0; j < 8; ++j) squares[8 * t + j] = __fmul_rn(o8[j], o8[j]);   // exact: BF16 squared fits FP32
    __syncthreads();
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = __fadd_rn(acc, squares[t + 256 * i]);
    partial[t] = acc;
    __syncthreads();
    if (t < 32) {
      // widths 128, 64, 32 fold four groups of 64 partials onto lane t, widths 16 .. 1 are lane shuffles
      float q = __fadd_rn(__fadd_rn(__fadd_rn(partial[t], partial[t + 128]), __fadd_rn(partial[t + 64], partial[t + 192])),
                          __fadd_rn(__fadd_rn(partial[t + 32], partial[t + 160]), __fadd_rn(partial[t + 96], partial[t + 224])));
#pragma unroll
      for (int width = 16; width >= 1; width >>= 1) q = __fadd_rn(q, __shfl_down_sync(0xffffffffu, q, width));
      if (t == 0) group_sums[0] = q;
    }
    __syncthreads();
    const float total = group_sums[0];
    const float inv = det_rsqrtf(__fadd_rn(__fdiv_rn(total, static_cast<float>(kHidden)), eps));
    float w[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(next_norm_weight) + t), w);
    uint32_t normed[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const float a = __fmul_rn(__fmul_rn(o8[j], inv), __fadd_rn(w[j], 1.0f));
      const float b = __fmul_rn(__fmul_rn(o8[j + 1], inv), __fadd_rn(w[j + 1], 1.0f));
      normed[j / 2] = static_cast<uint32_t>(float_to_bf16_bits(a)) |
                      (static_cast<uint32_t>(float_to_bf16_bits(b)) << 16);
    }
    reinterpret_cast<uint4*>(next_norm_out + base)[t] = make_uint4(normed[0], normed[1], normed[2], normed[3]);
  }
}


// ---------------------------------------------------------------------------
// Expert-parallel prefill over peer memory (NVLink).  Tokens are sharded T / W
// per GPU, experts 256 / W per GPU.  Everything that crosses NVLink is a plain
// store into a peer's exchange region: every rank's activation rows and routing
// go to every GPU (all-gathers by peer stores), and the weighted expert rows go
// to the GPU that owns their token -- from the down kernel's epilogue, or, in
// the pipelined variant, from the copy kernel below.  The tensor-core kernels
// only ever READ this GPU's own memory.
// ---------------------------------------------------------------------------
struct EpPointers {
  uint8_t* region[8];
};

// every rank's routing (ids, weights) into every rank's table, slot `rank`
__global__ void __launch_bounds__(256)
ep_publish_routing_kernel(const int32_t* __restrict__ ids, const float* __restrict__ weights, int n,
                          EpPointers peers, int world, int rank, size_t off_ids, size_t off_weights) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  const float w = weights[i];
  for (int q = 0; q < world; ++q) {
    reinterpret_cast<int32_t*>(peers.region[q] + off_ids)[static_cast<size_t>(rank) * n + i] = id;
    reinterpret_cast<float*>(peers.region[q] + off_weights)[static_cast<size_t>(rank) * n + i] = w;
  }
}

// every rank's h2 rows into every rank's [T, 2048] table, block `rank`: the all-gather that replaces a
// dispatch of single rows (with eight experts out of 256 per token nearly every rank needs nearly every
// token).  It does not depend on the routing, so it runs beside the router on its own stream; a small grid,
// since NVLink, not the SMs, sets its pace.
__global__ void __launch_bounds__(256)
ep_publish_rows_kernel(const uint4* __restrict__ rows, size_t n_vec, EpPointers peers, int world, int rank,
                       size_t off_h2) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    const uint4 v = rows[i];
    for (int q = 0; q < world; ++q)
      reinterpret_cast<uint4*>(peers.region[q] + off_h2)[static_cast<size_t>(rank) * n_vec + i] = v;
  }
}

// after the stores of the previous kernel: raise this rank's flag on every GPU
__global__ void ep_signal_kernel(EpPointers peers, int world, int rank, size_t off_flag, unsigned epoch) {
  const int q = threadIdx.x;
  if (q >= world) return;
  __threadfence_system();
  unsigned* flag = reinterpret_cast<unsigned*>(peers.region[q] + off_flag) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(flag), "r"(epoch) : "memory");
}

// bounded wait until every rank's flag in this GPU's region carries `epoch`
__global__ void ep_wait_kernel(const uint8_t* region, int world, size_t off_flag, unsigned epoch, int* status) {
  const int q = threadIdx.x;
  if (q >= world) return;
  const unsigned* flag = reinterpret_cast<const unsigned*>(region + off_flag) + q;
  const unsigned long long start = global_timer_ns();
  unsigned spins = 0;
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - epoch) >= 0) break;      // a later epoch also means this one has passed
    if ((++spins & 63u) == 0u && global_timer_ns() - start > kWaitBudgetNs) {
      atomicCAS(status, 0, kStatusTimeoutPeer);
      break;
    }
  }
}

// Sorted-row range of part `part` of `parts` of the plan's tiles (the same split the product kernel
// makes): tiles follow the sorted order, so a range of tiles is a range of rows.
__device__ __forceinline__ void part_rows(const int32_t* __restrict__ expert_offsets,
                                          const int32_t* __restrict__ tile_row0,
                                          const int32_t* __restrict__ tile_count, int part, int parts,
                                          int& row_lo, int& row_hi) {
  const int total = expert_offsets[kExperts];
  const int n_tiles = *tile_count;
  const int tile_lo = static_cast<int>(static_cast<long long>(n_tiles) * part / parts);
  const int tile_hi = static_cast<int>(static_cast<long long>(n_tiles) * (part + 1) / parts);
  row_lo = tile_lo < n_tiles ? tile_row0[tile_lo] : total;
  row_hi = tile_hi < n_tiles ? tile_row0[tile_hi] : total;
}

// dispatch: row `pos` of this GPU's plan <- h2 row of its token, wherever that token lives
__global__ void __launch_bounds__(256)
ep_gather_rows_kernel(EpPointers peers, size_t off_h2, int tokens_per_rank,
                      const int32_t* __restrict__ sorted_rows, const int32_t* __restrict__ expert_offsets,
                      const int32_t* __restrict__ tile_row0, const int32_t* __restrict__ tile_count,
                      int part, int parts, __nv_bfloat16* __restrict__ gathered) {
  const int lane = threadIdx.x & 31;
  int row_lo, row_hi;
  part_rows(expert_offsets, tile_row0, tile_count, part, parts, row_lo, row_hi);
  // a small grid that loops: the copy kernels share the SMs with the product kernels of another
  // part, whose one-block-per-SM grid must find room at once
  for (int pos = row_lo + blockIdx.x * 8 + (threadIdx.x >> 5); pos < row_hi; pos += gridDim.x * 8) {
    const int token = sorted_rows[pos] >> 3;
    const int owner = token / tokens_per_rank;
    const int local = token - owner * tokens_per_rank;
    const uint4* src = reinterpret_cast<const uint4*>(peers.region[owner] + off_h2) +
                       static_cast<size_t>(local) * (kHidden / 8);
    uint4* dst = reinterpret_cast<uint4*>(gathered + static_cast<size_t>(pos) * kHidden);
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = src[i * 32 + lane];
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[i * 32 + lane] = v[i];
  }
}

// combine, first half: the weighted expert output of plan row `pos` goes to the GPU that owns
// its token, at that token's (token, slot) position
__global__ void __launch_bounds__(256)
ep_return_rows_kernel(const __nv_bfloat16* __restrict__ expert_down, const int32_t* __restrict__ sorted_rows,
                      const int32_t* __restrict__ expert_offsets,
                      const int32_t* __restrict__ tile_row0, const int32_t* __restrict__ tile_count,
                      int part, int parts, EpPointers peers, size_t off_return, int tokens_per_rank) {
  const int lane = threadIdx.x & 31;
  int row_lo, row_hi;
  part_rows(expert_offsets, tile_row0, tile_count, part, parts, row_lo, row_hi);
  for (int pos = row_lo + blockIdx.x * 8 + (threadIdx.x >> 5); pos < row_hi; pos += gridDim.x * 8) {
    const int flat = sorted_rows[pos];
    const int owner = (flat >> 3) / tokens_per_rank;
    const int local_flat = flat - owner * tokens_per_rank * kTopK;
    const uint4* src = reinterpret_cast<const uint4*>(expert_down + static_cast<size_t>(pos) * kHidden);
    uint4* dst = reinterpret_cast<uint4*>(peers.region[owner] + off_return) +
                 static_cast<size_t>(local_flat) * (kHidden / 8);
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = src[i * 32 + lane];
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[i * 32 + lane] = v[i];
  }
}

// qualification view: weighted expert output rows in flat (token, slot) order
__global__ void __launch_bounds__(256)
export_slot_rows_kernel(const __nv_bfloat16* __restrict__ expert_down, const int32_t* __restrict__ row_position,
                        int routed_rows, __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int flat = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (flat >= routed_rows) return;
  const uint4* src = reinterpret_cast<const uint4*>(expert_down + static_cast<size_t>(row_position[flat]) * kHidden);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(flat) * kHidden);
#pragma unroll
  for (int i = 0; i < 8; ++i) dst[i * 32 + lane] = src[i * 32 + lane];
}

int set_error(char* error, size_t error_bytes, cudaError_t code, const char* what) {
  std::snprintf(error, error_bytes, "%s: %s (%s)", what, cudaGetErrorName(code),
                cudaGetErrorString(code));
  (void)cudaGetLastError();
  return static_cast<int>(code);
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

struct Layout {
  size_t ids, scores, weights, sigmoid, approx, stats, unit_counts, counts, offsets, sorted, position,
      tile_expert, tile_row0, tile_rows, tile_count, padded, gathered, act, down, shared_act,
      shared_scaled, x0, x1, h2, total;
};

Layout layout_for(size_t T) {
  Layout l{};
  size_t cursor = 0;
  auto take = [&](size_t bytes) { const size_t at = cursor; cursor += align256(bytes); return at; };
  const size_t rows = T * kTopK;
  const size_t units = (rows + kPlanRowsPerWarp - 1) / kPlanRowsPerWarp;
  const size_t tiles = static_cast<size_t>(max_tiles_for(static_cast<int>(T)));
  l.ids = take(rows * 4);
  l.scores = take(rows * 4);
  l.weights = take(rows * 4);
  l.sigmoid = take(T * 4);
  l.approx = take(T * kExperts * 4);
  l.stats = take(32);
  l.unit_counts = take(units * kExperts * 4);
  l.counts = take(kExperts * 4);
  l.offsets = take((kExperts + 1) * 4);
  l.sorted = take(rows * 4);
  l.position = take(rows * 4);
  l.tile_expert = take(tiles * 4);
  l.tile_row0 = take(tiles * 4);
  l.tile_rows = take(tiles * 4);
  l.tile_count = take(4);
  l.padded = take(4);
  l.gathered = take(rows * kHidden * 2);
  l.act = take(rows * kInter * 2);
  l.down = take(rows * kHidden * 2);
  l.shared_act = take(T * kSharedInter * 2);
  l.shared_scaled = take(T * kHidden * 2);
  l.x0 = take(T * kHidden * 2);
  l.x1 = take(T * kHidden * 2);
  l.h2 = take(T * kHidden * 2);
  l.total = cursor;
  return l;
}

}  // namespace

cudaError_t launch_router_row_norms(const __nv_bfloat16* router, float* norms, cudaStream_t stream) {
  router_row_norms_kernel<<<kExperts / 8, 256, 0, stream>>>(router, norms);
  return cudaGetLastError();
}

size_t prefill_workspace_bytes(uint32_t capacity_tokens) {
  return capacity_tokens == 0 ? 0 : layout_for(capacity_tokens).total;
}

int prefill_workspace_allocate(PrefillWorkspace* ws, uint32_t capacity_tokens, int sm_count,
                               char* error, size_t error_bytes) {
  const Layout l = layout_for(capacity_tokens);
  cudaError_t code = cudaMalloc(&ws->base, l.total);
  if (code != cudaSuccess) return set_error(error, error_bytes, code, "cudaMalloc prefill workspace");
  code = cudaMemset(ws->base, 0, l.total);
  if (code != cudaSuccess) return set_error(error, error_bytes, code, "cudaMemset prefill workspace");
  code = cudaStreamCreateWithFlags(&ws->side_stream, cudaStreamNonBlocking);
  if (code == cudaSuccess) code = cudaEventCreateWithFlags(&ws->fork_event, cudaEventDisableTiming);
  if (code == cudaSuccess) code = cudaEventCreateWithFlags(&ws->router_event, cudaEventDisableTiming);
  if (code == cudaSuccess) code = cudaEventCreateWithFlags(&ws->join_event, cudaEventDisableTiming);
  if (code == cudaSuccess) code = cudaStreamCreateWithFlags(&ws->inbound_stream, cudaStreamNonBlocking);
  if (code == cudaSuccess) code = cudaStreamCreateWithFlags(&ws->outbound_stream, cudaStreamNonBlocking);
  if (code == cudaSuccess) code = cudaEventCreateWithFlags(&ws->plan_event, cudaEventDisableTiming);
  if (code == cudaSuccess) code = cudaEventCreateWithFlags(&ws->returned_event, cudaEventDisableTiming);
  if (code == cudaSuccess) code = cudaEventCreateWithFlags(&ws->published_event, cudaEventDisableTiming);
  for (int k = 0; k < PrefillWorkspace::kMaxParts && code == cudaSuccess; ++k) {
    code = cudaEventCreateWithFlags(&ws->gathered_event[k], cudaEventDisableTiming);
    if (code == cudaSuccess) code = cudaEventCreateWithFlags(&ws->computed_event[k], cudaEventDisableTiming);
  }
  if (code != cudaSuccess) return set_error(error, error_bytes, code, "side stream / events of the prefill workspace");
  ws->total_bytes = l.total;
  ws->capacity = static_cast<int>(capacity_tokens);
  ws->sm_count = sm_count;
  uint8_t* b = ws->base;
  ws->topk_ids = reinterpret_cast<int32_t*>(b + l.ids);
  ws->topk_scores = reinterpret_cast<float*>(b + l.scores);
  ws->topk_weights = reinterpret_cast<float*>(b + l.weights);
  ws->shared_sigmoid = reinterpret_cast<float*>(b + l.sigmoid);
  ws->approx_logits = reinterpret_cast<float*>(b + l.approx);
  ws->router_stats = reinterpret_cast<int32_t*>(b + l.stats);
  ws->unit_counts = reinterpret_cast<int32_t*>(b + l.unit_counts);
  ws->expert_counts = reinterpret_cast<int32_t*>(b + l.counts);
  ws->expert_offsets = reinterpret_cast<int32_t*>(b + l.offsets);
  ws->sorted_rows = reinterpret_cast<int32_t*>(b + l.sorted);
  ws->row_position = reinterpret_cast<int32_t*>(b + l.position);
  ws->tile_expert = reinterpret_cast<int32_t*>(b + l.tile_expert);
  ws->tile_row0 = reinterpret_cast<int32_t*>(b + l.tile_row0);
  ws->tile_rows = reinterpret_cast<int32_t*>(b + l.tile_rows);
  ws->tile_count = reinterpret_cast<int32_t*>(b + l.tile_count);
  ws->padded_rows = reinterpret_cast<int32_t*>(b + l.padded);
  ws->gathered = reinterpret_cast<__nv_bfloat16*>(b + l.gathered);
  ws->expert_act = reinterpret_cast<__nv_bfloat16*>(b + l.act);
  ws->expert_down = reinterpret_cast<__nv_bfloat16*>(b + l.down);
  ws->shared_act = reinterpret_cast<__nv_bfloat16*>(b + l.shared_act);
  ws->shared_scaled = reinterpret_cast<__nv_bfloat16*>(b + l.shared_scaled);
  ws->stack_x0 = reinterpret_cast<__nv_bfloat16*>(b + l.x0);
  ws->stack_x1 = reinterpret_cast<__nv_bfloat16*>(b + l.x1);
  ws->stack_h2 = reinterpret_cast<__nv_bfloat16*>(b + l.h2);
  return AIMA_MOE_OK;
}

void prefill_workspace_free(PrefillWorkspace* ws) {
  if (ws->base != nullptr) cudaFree(ws->base);
  if (ws->fork_event != nullptr) cudaEventDestroy(ws->fork_event);
  if (ws->router_event != nullptr) cudaEventDestroy(ws->router_event);
  if (ws->join_event != nullptr) cudaEventDestroy(ws->join_event);
  if (ws->side_stream != nullptr) cudaStreamDestroy(ws->side_stream);
  if (ws->plan_event != nullptr) cudaEventDestroy(ws->plan_event);
  if (ws->returned_event != nullptr) cudaEventDestroy(ws->returned_event);
  if (ws->published_event != nullptr) cudaEventDestroy(ws->published_event);
  for (int k = 0; k < PrefillWorkspace::kMaxParts; ++k) {
    if (ws->gathered_event[k] != nullptr) cudaEventDestroy(ws->gathered_event[k]);
    if (ws->computed_event[k] != nullptr) cudaEventDestroy(ws->computed_event[k]);
  }
  if (ws->inbound_stream != nullptr) cudaStreamDestroy(ws->inbound_stream);
  if (ws->outbound_stream != nullptr) cudaStreamDestroy(ws->outbound_stream);
  *ws = PrefillWorkspace{};
}

// Qualification: routing supplied by the harness replaces the router's ids and weights (the router still
// runs: the shared expert's sigmoid gate comes from it).  Mirrors the reference's "oracle-seeded
// routing" rerun (native/src/native_moe_prefill.hip.cpp:1059-1123), which isolates the expert
// arithmetic from tie-order effects.
__global__ void forced_routing_kernel(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ weights,
                                      int n, int32_t* __restrict__ topk_ids, float* __restrict__ topk_weights,
                                      float* __restrict__ topk_scores) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  topk_ids[i] = (id >= 0 && id < kExperts) ? id : 0;
  topk_weights[i] = __bfloat162float(weights[i]);
  topk_scores[i] = 0.0f;
}

int prefill_layer_launch(PrefillWorkspace* ws, const PrefillCall& call, cudaStream_t stream,
                         int* launches, char* error, size_t error_bytes) {
  const int T = call.tokens;
  const PdlScope pdl_scope(T <= pdl_max_tokens());
  const int rows = T * kTopK;
  const aima_moe_debug_views* dbg = call.debug;
  int count = 0;
  cudaError_t code;

  // fork: the shared gate/up product needs only h2
  cudaStream_t side = ws->side_stream;
  if ((code = cudaEventRecord(ws->fork_event, stream)) != cudaSuccess ||
      (code = cudaStreamWaitEvent(side, ws->fork_event, 0)) != cudaSuccess)
    return set_error(error, error_bytes, code, "fork of the shared-expert stream");
  auto product = [&](GemmMode mode, const GroupedGemm& problem, const TcExtra& x, cudaStream_t on) {
    return ws->use_simt_gemm ? launch_grouped_gemm_simt(mode, problem, on)
                             : launch_grouped_gemm_tc(mode, problem, x, on);
  };
  GroupedGemm s{};
  TcExtra shared_extra{};
  shared_extra.status = ws->status; shared_extra.sm_count = ws->sm_count;
  s.tile_expert = nullptr; s.tile_row0 = nullptr; s.tile_rows = nullptr; s.tile_count = nullptr;
  s.max_tiles = (T + kTileRows - 1) / kTileRows; s.dense_rows = T;
  s.a = static_cast<const __nv_bfloat16*>(call.h2); s.lda = kHidden; s.k = kHidden;
  s.b0 = call.layer.shared_gate_proj; s.b1 = call.layer.shared_up_proj; s.b_expert_stride = 0;
  s.n = kSharedInter; s.c = ws->shared_act; s.ldc = kSharedInter;
  shared_extra.a_rows = static_cast<uint64_t>(T); shared_extra.experts_in_b = 1;
  if ((code = product(kGemmSharedGateUp, s, shared_extra, side)) != cudaSuccess)
    return set_error(error, error_bytes, code, "grouped gemm shared gate_up");
  ++count;

  const bool exact_router = ws->exact_router || (dbg != nullptr && dbg->router_logits != nullptr) ||
                            call.router_row_norms == nullptr;
  if (exact_router) {
    code = opt_in_dynamic_smem<prefill_router_kernel>(kRouterSmemBytes);
    if (code != cudaSuccess) return set_error(error, error_bytes, code, "cudaFuncSetAttribute router");
    prefill_router_kernel<<<(T + kRouterWarps - 1) / kRouterWarps, kRouterWarps * 32, kRouterSmemBytes, stream>>>(
        static_cast<const __nv_bfloat16*>(call.h2), call.layer.router, call.layer.shared_gate,
        call.router_bias, call.quant_eighths, T, ws->topk_ids, ws->topk_scores, ws->topk_weights,
        ws->shared_sigmoid, dbg ? static_cast<float*>(dbg->router_logits) : nullptr,
        dbg ? static_cast<__nv_bfloat16*>(dbg->topk_weights) : nullptr);
    if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "prefill_router_kernel");
    ++count;
  } else {
    // tensor-core logits for the candidate filter, then exact recomputation of the candidates
    GroupedGemm r{};
    r.max_tiles = (T + kTileRows - 1) / kTileRows; r.dense_rows = T;
    r.a = static_cast<const __nv_bfloat16*>(call.h2); r.lda = kHidden; r.k = kHidden;
    r.b0 = call.layer.router; r.n = kExperts; r.c_f32 = ws->approx_logits; r.ldc = kExperts;
    TcExtra rx{};
    rx.status = ws->status; rx.sm_count = ws->sm_count; rx.a_rows = static_cast<uint64_t>(T); rx.experts_in_b = 1;
    if ((code = launch_grouped_gemm_tc(kGemmPlainF32, r, rx, stream)) != cudaSuccess)
      return set_error(error, error_bytes, code, "router logits product");
    code = launch_pdl(prefill_router_certified_kernel, dim3((T + kCertWarps - 1) / kCertWarps), dim3(kCertWarps * 32),
                      0, stream, static_cast<const __nv_bfloat16*>(call.h2), call.layer.router,
                      call.layer.shared_gate, ws->approx_logits, call.router_row_norms, call.router_bias,
                      call.quant_eighths, T, ws->topk_ids, ws->topk_scores, ws->topk_weights, ws->shared_sigmoid,
                      dbg ? static_cast<__nv_bfloat16*>(dbg->topk_weights) : nullptr, ws->router_stats, ws->router_audit_stride);
    if (code != cudaSuccess)
      return set_error(error, error_bytes, code, "prefill_router_certified_kernel");
    count += 2;
  }

  if (call.forced_ids != nullptr) {
    forced_routing_kernel<<<(rows + 255) / 256, 256, 0, stream>>>(
        call.forced_ids, static_cast<const __nv_bfloat16*>(call.forced_weights), rows, ws->topk_ids,
        ws->topk_weights, ws->topk_scores);
    if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "forced_routing_kernel");
    ++count;
  }

  // the shared down product scales by the sigmoid the router kernel wrote
  if ((code = cudaEventRecord(ws->router_event, stream)) != cudaSuccess ||
      (code = cudaStreamWaitEvent(side, ws->router_event, 0)) != cudaSuccess)
    return set_error(error, error_bytes, code, "router event of the shared-expert stream");
  s.a = ws->shared_act; s.lda = kSharedInter; s.k = kSharedInter;
  s.b0 = call.layer.shared_down_proj; s.b1 = nullptr;
  s.n = kHidden; s.c = ws->shared_scaled; s.ldc = kHidden;
  s.row_scale = ws->shared_sigmoid;
  shared_extra.a_rows = static_cast<uint64_t>(ws->capacity);
  if ((code = product(kGemmSharedDown, s, shared_extra, side)) != cudaSuccess)
    return set_error(error, error_bytes, code, "grouped gemm shared down");
  ++count;
  if ((code = cudaEventRecord(ws->join_event, side)) != cudaSuccess)
    return set_error(error, error_bytes, code, "join event of the shared-expert stream");

  // Expert products: one block per 128-row tile; the two-SM form (a pair of blocks per 256-row tile) behind a
  // flag.  Both stream every expert's weights once at T = 8192 and are bound by that stream -- 302 / 170 us
  // (gate_up / down) against 308 / 218 us for the pair with materialised rows, and the pair's row gather has to
  // cross to the leader's barrier, which doubles its gate_up time -- so the simpler form is the default.
  const bool pair_products = ws->pair_products && !ws->use_simt_gemm;
  if ((code = launch_plan(ws, ws->topk_ids, rows, 0, kExperts, stream, &count, pair_products ? 2 * kTileRows : kTileRows)) !=
      cudaSuccess)
    return set_error(error, error_bytes, code, "dispatch plan");

  // Dispatch is fused into the gate_up kernel: two of its warps fetch each tile's rows by token index
  // with asynchronous 16-byte copies (0.689 vs 0.745 ms per T = 8192 layer).  The materialised copy in
  // expert order, read by tiled TMA loads, remains for the CUDA-core cross-check and behind a flag.
  const bool fused_dispatch = ws->fused_dispatch && !ws->use_simt_gemm;
  if (!fused_dispatch) {
    gather_rows_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(call.h2), ws->sorted_rows, rows, ws->gathered);
    if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "gather_rows_kernel");
    ++count;
  }

  // routed experts: gate_up + SwiGLU, then down x routing weight
  GroupedGemm g{};
  g.tile_expert = ws->tile_expert; g.tile_row0 = ws->tile_row0; g.tile_rows = ws->tile_rows;
  g.tile_count = ws->tile_count; g.max_tiles = max_tiles_for(T); g.dense_rows = 0;
  g.a = ws->gathered; g.lda = kHidden; g.k = kHidden;
  g.b0 = call.layer.expert_gate_up; g.b1 = nullptr;
  g.b_expert_stride = static_cast<size_t>(2 * kInter) * kHidden;
  g.n = kInter; g.c = ws->expert_act; g.ldc = kInter;
  g.row_scale = nullptr; g.sorted_rows = ws->sorted_rows;
  TcExtra extra{};
  extra.status = ws->status; extra.sm_count = ws->sm_count;
  extra.experts_in_b = call.experts_local;
  extra.pair = pair_products;
  if (fused_dispatch) {
    g.gather_src = static_cast<const __nv_bfloat16*>(call.h2);
    extra.a_rows = static_cast<uint64_t>(T);
  } else {
    extra.a_rows = static_cast<uint64_t>(ws->capacity) * kTopK;
  }
  if ((code = product(kGemmExpertGateUp, g, extra, stream)) != cudaSuccess)
    return set_error(error, error_bytes, code, "grouped gemm expert gate_up");
  g.gather_src = nullptr;
  extra.a_rows = static_cast<uint64_t>(ws->capacity) * kTopK;
  g.a = ws->expert_act; g.lda = kInter; g.k = kInter;
  g.b0 = call.layer.expert_down; g.b_expert_stride = static_cast<size_t>(kHidden) * kInter;
  g.n = kHidden; g.c = ws->expert_down; g.ldc = kHidden;
  g.row_scale = ws->topk_weights; g.sorted_rows = ws->sorted_rows;
  if ((code = product(kGemmExpertDown, g, extra, stream)) != cudaSuccess)
    return set_error(error, error_bytes, code, "grouped gemm expert down");
  count += 2;

  // join: the combine needs the shared expert's output
  if ((code = cudaStreamWaitEvent(stream, ws->join_event, 0)) != cudaSuccess)
    return set_error(error, error_bytes, code, "join of the shared-expert stream");
  combine_kernel<<<T, 256, 0, stream>>>(ws->expert_down, ws->row_position, ws->shared_scaled,
                                        static_cast<const __nv_bfloat16*>(call.residual),
                                        static_cast<__nv_bfloat16*>(call.out),
                                        dbg ? static_cast<__nv_bfloat16*>(dbg->routed) : nullptr,
                                        static_cast<const __nv_bfloat16*>(call.next_norm_weight),
                                        static_cast<__nv_bfloat16*>(call.next_norm_out), call.eps);
  if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "combine_kernel");
  ++count;

  if (dbg != nullptr) {
    auto copy = [&](void* dst, const void* src, size_t bytes) {
      if (dst != nullptr) return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
      return cudaSuccess;
    };
    code = copy(dbg->h2, call.h2, static_cast<size_t>(T) * kHidden * 2);
    if (code == cudaSuccess) code = copy(dbg->topk_ids, ws->topk_ids, static_cast<size_t>(rows) * 4);
    if (code == cudaSuccess) code = copy(dbg->topk_scores, ws->topk_scores, static_cast<size_t>(rows) * 4);
    if (code == cudaSuccess) code = copy(dbg->shared_scaled, ws->shared_scaled, static_cast<size_t>(T) * kHidden * 2);
    if (code == cudaSuccess) code = copy(dbg->expert_counts, ws->expert_counts, kExperts * 4);
    if (code == cudaSuccess) code = copy(dbg->expert_offsets, ws->expert_offsets, (kExperts + 1) * 4);
    if (code == cudaSuccess) code = copy(dbg->sorted_rows, ws->sorted_rows, static_cast<size_t>(rows) * 4);
    if (code != cudaSuccess) return set_error(error, error_bytes, code, "cudaMemcpyAsync debug views");
    if (dbg->slot_rows != nullptr) {
      export_slot_rows_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(ws->expert_down, ws->row_position, rows,
                                                                  static_cast<__nv_bfloat16*>(dbg->slot_rows));
      if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "export_slot_rows_kernel");
    }
  }
  *launches = count;
  return AIMA_MOE_OK;
}

size_t ep_prefill_region_bytes(int capacity_tokens, int world, EpPrefillLayout* layout) {
  // capacity_tokens = global tokens per call; every rank holds capacity / world of them at most,
  // but the tables are sized for the global count so that any split fits
  const size_t rows = static_cast<size_t>(capacity_tokens) * kTopK;
  size_t cursor = 0;
  auto take = [&](size_t bytes) { const size_t at = cursor; cursor += (bytes + 255) / 256 * 256; return at; };
  EpPrefillLayout l{};
  l.off_flags_routing = take(64);
  l.off_flags_returned = take(64);
  l.off_ids = take(rows * 4);
  l.off_weights = take(rows * 4);
  l.off_h2 = take(static_cast<size_t>(capacity_tokens) * kHidden * 2);
  l.off_return = take(rows * kHidden * 2);
  l.bytes = cursor;
  (void)world;
  if (layout != nullptr) *layout = l;
  return cursor;
}

int prefill_layer_launch_ep(PrefillWorkspace* ws, const PrefillCall& call, EpPrefill* ep,
                            cudaStream_t stream, int* launches, char* error, size_t error_bytes) {
  const int T_loc = call.tokens;
  const PdlScope pdl_scope(false);   // plain stream order: kernels of this path wait for peers, nothing may sit resident ahead of them
  const int W = ep->world;
  const int T = T_loc * W;
  const int rows_loc = T_loc * kTopK;
  const int rows = T * kTopK;
  const aima_moe_debug_views* dbg = call.debug;
  const EpPrefillLayout& L = ep->layout;
  EpPointers peers{};
  for (int q = 0; q < W; ++q) peers.region[q] = ep->peers[q];
  uint8_t* mine = ep->peers[ep->rank];
  const unsigned epoch = ++ep->epoch;
  int count = 0;
  cudaError_t code;
  int mark_index = 0;
  auto mark = [&]() {
    if (ep->trace && ep->stage_events[mark_index] != nullptr) cudaEventRecord(ep->stage_events[mark_index], stream);
    ++mark_index;
  };
  mark();

  // The shared expert (weights replicated, this rank's tokens) runs on the side stream: its gate/up
  // product starts at once, its down product once the router kernel has written the sigmoid; it
  // fills the SMs while the main stream waits for peers and for rows crossing NVLink.
  cudaStream_t side = ws->side_stream;
  if ((code = cudaEventRecord(ws->fork_event, stream)) != cudaSuccess ||
      (code = cudaStreamWaitEvent(side, ws->fork_event, 0)) != cudaSuccess)
    return set_error(error, error_bytes, code, "fork of the shared-expert stream");
  GroupedGemm s{};
  TcExtra shared_extra{};
  shared_extra.status = ws->status; shared_extra.sm_count = ws->sm_count;
  s.max_tiles = (T_loc + kTileRows - 1) / kTileRows; s.dense_rows = T_loc;
  s.a = static_cast<const __nv_bfloat16*>(call.h2); s.lda = kHidden; s.k = kHidden;
  s.b0 = call.layer.shared_gate_proj; s.b1 = call.layer.shared_up_proj;
  s.n = kSharedInter; s.c = ws->shared_act; s.ldc = kSharedInter;
  shared_extra.a_rows = static_cast<uint64_t>(T_loc); shared_extra.experts_in_b = 1;
  if ((code = launch_grouped_gemm_tc(kGemmSharedGateUp, s, shared_extra, side)) != cudaSuccess)
    return set_error(error, error_bytes, code, "grouped gemm shared gate_up");
  ++count;

  // 0. this rank's h2 rows to every GPU, on the inbound stream beside the router (the flags of step 2 cover it)
  if ((code = cudaStreamWaitEvent(ws->inbound_stream, ws->fork_event, 0)) != cudaSuccess)
    return set_error(error, error_bytes, code, "fork of the row all-gather");
  ep_publish_rows_kernel<<<96, 256, 0, ws->inbound_stream>>>(
      static_cast<const uint4*>(call.h2), static_cast<size_t>(T_loc) * (kHidden / 8), peers, W, ep->rank, L.off_h2);
  if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "ep_publish_rows_kernel");
  ++count;
  if ((code = cudaEventRecord(ws->published_event, ws->inbound_stream)) != cudaSuccess)
    return set_error(error, error_bytes, code, "published event");

  // 1. route this rank's tokens (certified router)
  GroupedGemm r{};
  r.max_tiles = (T_loc + kTileRows - 1) / kTileRows; r.dense_rows = T_loc;
  r.a = static_cast<const __nv_bfloat16*>(call.h2); r.lda = kHidden; r.k = kHidden;
  r.b0 = call.layer.router; r.n = kExperts; r.c_f32 = ws->approx_logits; r.ldc = kExperts;
  TcExtra rx{};
  rx.status = ws->status; rx.sm_count = ws->sm_count; rx.a_rows = static_cast<uint64_t>(T_loc); rx.experts_in_b = 1;
  if ((code = launch_grouped_gemm_tc(kGemmPlainF32, r, rx, stream)) != cudaSuccess)
    return set_error(error, error_bytes, code, "router logits product");
  prefill_router_certified_kernel<<<(T_loc + kCertWarps - 1) / kCertWarps, kCertWarps * 32, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(call.h2), call.layer.router, call.layer.shared_gate,
      ws->approx_logits, call.router_row_norms, call.router_bias, call.quant_eighths, T_loc, ws->topk_ids,
      ws->topk_scores, ws->topk_weights, ws->shared_sigmoid,
      dbg ? static_cast<__nv_bfloat16*>(dbg->topk_weights) : nullptr, ws->router_stats, ws->router_audit_stride);
  if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "prefill_router_certified_kernel");
  count += 2;
  if ((code = cudaEventRecord(ws->router_event, stream)) != cudaSuccess ||
      (code = cudaStreamWaitEvent(side, ws->router_event, 0)) != cudaSuccess)
    return set_error(error, error_bytes, code, "router event of the shared-expert stream");
  s.a = ws->shared_act; s.lda = kSharedInter; s.k = kSharedInter;
  s.b0 = call.layer.shared_down_proj; s.b1 = nullptr;
  s.n = kHidden; s.c = ws->shared_scaled; s.ldc = kHidden; s.row_scale = ws->shared_sigmoid;
  shared_extra.a_rows = static_cast<uint64_t>(ws->capacity);
  if ((code = launch_grouped_gemm_tc(kGemmSharedDown, s, shared_extra, side)) != cudaSuccess)
    return set_error(error, error_bytes, code, "grouped gemm shared down");
  ++count;
  if ((code = cudaEventRecord(ws->join_event, side)) != cudaSuccess)
    return set_error(error, error_bytes, code, "join event of the shared-expert stream");

  mark();
  // 2. all-gather of the routing tables by peer stores, then flags
  ep_publish_routing_kernel<<<(rows_loc + 255) / 256, 256, 0, stream>>>(
      ws->topk_ids, ws->topk_weights, rows_loc, peers, W, ep->rank, L.off_ids, L.off_weights);
  if ((code = cudaStreamWaitEvent(stream, ws->published_event, 0)) != cudaSuccess)
    return set_error(error, error_bytes, code, "join of the row all-gather");
  ep_signal_kernel<<<1, 32, 0, stream>>>(peers, W, ep->rank, L.off_flags_routing, epoch);
  ep_wait_kernel<<<1, 32, 0, stream>>>(mine, W, L.off_flags_routing, epoch, ws->status);
  if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "routing exchange");
  count += 3;
  const int32_t* ids_all = reinterpret_cast<const int32_t*>(mine + L.off_ids);
  const float* weights_all = reinterpret_cast<const float*>(mine + L.off_weights);

  mark();
  // 3. plan over the global rows that land on this GPU's experts
  const int expert_lo = ep->rank * call.experts_local;
  const int expert_hi = expert_lo + call.experts_local;
  if ((code = launch_plan(ws, ids_all, rows, expert_lo, expert_hi, stream, &count)) != cudaSuccess)
    return set_error(error, error_bytes, code, "dispatch plan");

  mark();
  // 4.-6. dispatch, products and row return, pipelined over `parts` ranges of the plan's tiles:
  //   inbound stream   rows of part k copied from this GPU's table of all activations into expert order
  //   caller's stream  gate_up and down products of part k once its rows are here
  //   outbound stream  weighted rows of part k stored to the GPUs that own their tokens
  const int parts = ws->ep_parts >= 1 && ws->ep_parts <= PrefillWorkspace::kMaxParts ? ws->ep_parts : 1;
  // Row return: with one part the down kernel stores its rows to their owners itself (fused_return); with the
  // pipeline a copy kernel on the outbound stream sends the rows of part k while part k + 1 is computed.
  const bool fused_return = parts == 1 && ws->ep_fused_return;
  // Dispatch: all rows are in this GPU's table since the flags of step 2, in global token order, so with one
  // part the gate_up kernel gathers them itself as on one GPU; otherwise a copy kernel puts them in expert order.
  const bool fused_dispatch = parts == 1 && ws->ep_fused_dispatch;
  EpPointers local_blocks{};      // block q of this GPU's table: the tokens of rank q
  for (int q = 0; q < W; ++q) local_blocks.region[q] = mine + static_cast<size_t>(q) * T_loc * kHidden * 2;
  const int part_blocks = min(((max_tiles_for(T) / parts + 1) * kTileRows + 7) / 8, 2 * ws->sm_count);
  cudaStream_t inbound = ws->inbound_stream, outbound = ws->outbound_stream;
  if ((code = cudaEventRecord(ws->plan_event, stream)) != cudaSuccess ||
      (code = cudaStreamWaitEvent(inbound, ws->plan_event, 0)) != cudaSuccess ||
      (code = cudaStreamWaitEvent(outbound, ws->plan_event, 0)) != cudaSuccess)
    return set_error(error, error_bytes, code, "fork of the dispatch / return streams");
  for (int k = 0; k < parts && !fused_dispatch; ++k) {
    ep_gather_rows_kernel<<<part_blocks, 256, 0, inbound>>>(local_blocks, L.off_h2, T_loc, ws->sorted_rows,
                                                            ws->expert_offsets, ws->tile_row0, ws->tile_count,
                                                            k, parts, ws->gathered);
    if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "ep_gather_rows_kernel");
    if ((code = cudaEventRecord(ws->gathered_event[k], inbound)) != cudaSuccess)
      return set_error(error, error_bytes, code, "gathered event");
    ++count;
  }
  GroupedGemm g{};
  g.tile_expert = ws->tile_expert; g.tile_row0 = ws->tile_row0; g.tile_rows = ws->tile_rows;
  g.tile_count = ws->tile_count; g.max_tiles = max_tiles_for(T); g.dense_rows = 0;
  g.expert_base = expert_lo;
  g.parts = parts;
  TcExtra extra{};
  extra.status = ws->status; extra.sm_count = ws->sm_count;
  extra.a_rows = static_cast<uint64_t>(ws->capacity) * kTopK; extra.experts_in_b = call.experts_local;
  for (int k = 0; k < parts; ++k) {
    if (!fused_dispatch && (code = cudaStreamWaitEvent(stream, ws->gathered_event[k], 0)) != cudaSuccess)
      return set_error(error, error_bytes, code, "wait for gathered rows");
    if (k == 0) mark();
    g.part = k;
    g.a = ws->gathered; g.lda = kHidden; g.k = kHidden;
    g.gather_src = fused_dispatch ? reinterpret_cast<const __nv_bfloat16*>(mine + L.off_h2) : nullptr;
    extra.a_rows = fused_dispatch ? static_cast<uint64_t>(T) : static_cast<uint64_t>(ws->capacity) * kTopK;
    g.b0 = call.layer.expert_gate_up; g.b_expert_stride = static_cast<size_t>(2 * kInter) * kHidden;
    g.n = kInter; g.c = ws->expert_act; g.ldc = kInter;
    g.row_scale = nullptr; g.sorted_rows = ws->sorted_rows;
    if ((code = launch_grouped_gemm_tc(kGemmExpertGateUp, g, extra, stream)) != cudaSuccess)
      return set_error(error, error_bytes, code, "grouped gemm expert gate_up");
    g.gather_src = nullptr;
    extra.a_rows = static_cast<uint64_t>(ws->capacity) * kTopK;
    g.a = ws->expert_act; g.lda = kInter; g.k = kInter;
    g.b0 = call.layer.expert_down; g.b_expert_stride = static_cast<size_t>(kHidden) * kInter;
    g.n = kHidden; g.c = ws->expert_down; g.ldc = kHidden;
    g.row_scale = weights_all;
    if (fused_return) {
      // the down kernel's epilogue stores every weighted row where its token lives
      for (int q = 0; q < W; ++q) g.scatter_region[q] = ep->peers[q];
      g.scatter_offset = L.off_return;
      g.scatter_tokens_per_rank = T_loc;
    }
    if ((code = launch_grouped_gemm_tc(kGemmExpertDown, g, extra, stream)) != cudaSuccess)
      return set_error(error, error_bytes, code, "grouped gemm expert down");
    count += 2;
    if (fused_return) break;
    if ((code = cudaEventRecord(ws->computed_event[k], stream)) != cudaSuccess ||
        (code = cudaStreamWaitEvent(outbound, ws->computed_event[k], 0)) != cudaSuccess)
      return set_error(error, error_bytes, code, "computed event");
    ep_return_rows_kernel<<<part_blocks, 256, 0, outbound>>>(ws->expert_down, ws->sorted_rows, ws->expert_offsets,
                                                             ws->tile_row0, ws->tile_count, k, parts, peers,
                                                             L.off_return, T_loc);
    if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "ep_return_rows_kernel");
    ++count;
  }
  mark();
  // all rows stored: raise this rank's flag on every GPU, then rejoin the caller's stream
  ep_signal_kernel<<<1, 32, 0, fused_return ? stream : outbound>>>(peers, W, ep->rank, L.off_flags_returned, epoch);
  if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "row return");
  ++count;
  if (!fused_return &&
      ((code = cudaEventRecord(ws->returned_event, outbound)) != cudaSuccess ||
       (code = cudaStreamWaitEvent(stream, ws->returned_event, 0)) != cudaSuccess))
    return set_error(error, error_bytes, code, "join of the return stream");

  mark();
  // 7. the shared expert's output is needed from here on
  if ((code = cudaStreamWaitEvent(stream, ws->join_event, 0)) != cudaSuccess)
    return set_error(error, error_bytes, code, "join of the shared-expert stream");

  // 8. combine, second half: wait for all eight rows of every local token, sum, add
  ep_wait_kernel<<<1, 32, 0, stream>>>(mine, W, L.off_flags_returned, epoch, ws->status);
  combine_kernel<<<T_loc, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(mine + L.off_return), nullptr,
                                            ws->shared_scaled, static_cast<const __nv_bfloat16*>(call.residual),
                                            static_cast<__nv_bfloat16*>(call.out),
                                            dbg ? static_cast<__nv_bfloat16*>(dbg->routed) : nullptr,
                                            static_cast<const __nv_bfloat16*>(call.next_norm_weight),
                                            static_cast<__nv_bfloat16*>(call.next_norm_out), call.eps);
  if ((code = cudaGetLastError()) != cudaSuccess) return set_error(error, error_bytes, code, "combine_kernel");
  count += 2;
  mark();
  if (dbg != nullptr) {
    auto copy = [&](void* dst, const void* src, size_t bytes) {
      if (dst != nullptr) return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream);
      return cudaSuccess;
    };
    code = copy(dbg->topk_ids, ws->topk_ids, static_cast<size_t>(rows_loc) * 4);
    if (code == cudaSuccess) code = copy(dbg->topk_scores, ws->topk_scores, static_cast<size_t>(rows_loc) * 4);
    if (code == cudaSuccess) code = copy(dbg->shared_scaled, ws->shared_scaled, static_cast<size_t>(T_loc) * kHidden * 2);
    if (code == cudaSuccess) code = copy(dbg->expert_counts, ws->expert_counts, kExperts * 4);
    if (code != cudaSuccess) return set_error(error, error_bytes, code, "cudaMemcpyAsync debug views");
  }
  *launches = count;
  return AIMA_MOE_OK;
}

}  // namespace aima
