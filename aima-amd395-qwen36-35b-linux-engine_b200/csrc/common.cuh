// Shared device helpers of the B200 MoE provider: model constants, BF16
// conversion, the deterministic arithmetic contract (dot product order, exp,
// reciprocal square root) and bounded waits.
//
// The arithmetic contract is what makes routing bit-exact between this library
// and its CPU checker: every FP32 reduction on the routing path has ONE fixed
// order, written with explicit round-to-nearest intrinsics so that the compiler
// can neither re-associate nor contract differently from the C restatement.
#pragma once

#include <cstdlib>
#include <mutex>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace aima {

constexpr int kHidden = 2048;
constexpr int kExperts = 256;
constexpr int kTopK = 8;
constexpr int kInter = 512;        // expert intermediate; gate_up has 2*kInter rows
constexpr int kSharedInter = 512;
constexpr int kMaxLayers = 64;

// Device status word values (0 = healthy).
constexpr int kStatusOk = 0;
constexpr int kStatusTimeoutGridBarrier = 1;
constexpr int kStatusTimeoutMbarrier = 2;
constexpr int kStatusTimeoutIds = 3;
constexpr int kStatusTimeoutPeer = 4;
constexpr int kStatusBadExpert = 5;

// Budget of every device-side wait, in nanoseconds of %globaltimer.
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;

struct LayerPtrs {
  const __nv_bfloat16* router;            // [256, 2048]
  const __nv_bfloat16* expert_gate_up;    // [E_local, 1024, 2048]
  const __nv_bfloat16* expert_down;       // [E_local, 2048, 512]
  const __nv_bfloat16* shared_gate;       // [1, 2048]
  const __nv_bfloat16* shared_gate_proj;  // [512, 2048]
  const __nv_bfloat16* shared_up_proj;    // [512, 2048]
  const __nv_bfloat16* shared_down_proj;  // [2048, 512]
  const __nv_bfloat16* norm_weight;       // [2048] or nullptr
};

// ---------------------------------------------------------------------------
// BF16 <-> FP32
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t packed) {
  return __uint_as_float(packed << 16);
}
__device__ __forceinline__ float bf16_hi(uint32_t packed) {
  return __uint_as_float(packed & 0xffff0000u);
}
__device__ __forceinline__ float bf16_bits_to_float(uint16_t bits) {
  return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}
__device__ __forceinline__ uint16_t float_to_bf16_bits(float value) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(value));
}
__device__ __forceinline__ float round_bf16(float value) {
  return __bfloat162float(__float2bfloat16_rn(value));
}

// ---------------------------------------------------------------------------
// Deterministic transcendental functions (same operations as the C checker).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float det_expf(float x) {
  x = fminf(fmaxf(x, -87.0f), 88.0f);
  const float t = __fmul_rn(x, 1.44269504088896341f);
  const float n = rintf(t);
  float r = __fmaf_rn(n, -0.693145751953125f, x);
  r = __fmaf_rn(n, -1.42860682030941723e-06f, r);
  float p = 1.0f / 720.0f;
  p = __fmaf_rn(p, r, 1.0f / 120.0f);
  p = __fmaf_rn(p, r, 1.0f / 24.0f);
  p = __fmaf_rn(p, r, 1.0f / 6.0f);
  p = __fmaf_rn(p, r, 0.5f);
  p = __fmaf_rn(p, r, 1.0f);
  p = __fmaf_rn(p, r, 1.0f);
  const int e = static_cast<int>(n) + 127;
  return __fmul_rn(p, __int_as_float(e << 23));
}
__device__ __forceinline__ float det_silu(float g) {
  return __fdiv_rn(g, __fadd_rn(1.0f, det_expf(-g)));
}
__device__ __forceinline__ float det_sigmoid(float g) {
  return __fdiv_rn(1.0f, __fadd_rn(1.0f, det_expf(-g)));
}
// Correctly rounded FP32 reciprocal square root up to double rounding:
// IEEE double sqrt and divide, one conversion.
__device__ __forceinline__ float det_rsqrtf(float v) {
  return static_cast<float>(__ddiv_rn(1.0, __dsqrt_rn(static_cast<double>(v))));
}

// ---------------------------------------------------------------------------
// Canonical warp dot product.
// Lane l owns every 8-element group g with g % 32 == l.  Its partial sum runs
// over its groups in ascending order, 8 fused multiply-adds per group; the 32
// partials are merged with the xor butterfly 16, 8, 4, 2, 1, after which all
// lanes hold the same value.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float butterfly_sum(float v) {
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) {
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, s));
  }
  return v;
}

// Eight canonical warp reductions at once.  v[d] is this lane's partial of sum d;
// the result is the butterfly (16, 8, 4, 2, 1) total of sum d(lane), with
// d(lane) = 4 * bit4 + 2 * bit3 + bit2 of the lane index.  Each level pairs the
// same lanes as butterfly_sum, so the bits are identical, with 9 shuffles
// instead of 40.
__device__ __forceinline__ float warp_reduce8(const float* v, int lane) {
  const bool b4 = (lane & 16) != 0, b3 = (lane & 8) != 0, b2 = (lane & 4) != 0;
  float a[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float keep = b4 ? v[j + 4] : v[j];
    const float send = b4 ? v[j] : v[j + 4];
    a[j] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 16));
  }
  float b[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float keep = b3 ? a[j + 2] : a[j];
    const float send = b3 ? a[j] : a[j + 2];
    b[j] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 8));
  }
  const float keep = b2 ? b[1] : b[0];
  const float send = b2 ? b[0] : b[1];
  float c = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 4));
  c = __fadd_rn(c, __shfl_xor_sync(0xffffffffu, c, 2));
  c = __fadd_rn(c, __shfl_xor_sync(0xffffffffu, c, 1));
  return c;
}
__device__ __forceinline__ int reduce8_slot(int lane) {
  return ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
}


// Sum of squares of a 2048-wide row in the order of the reference's RMSNorm kernels
// (native/src/native_pointwise.hip.cpp:109-142): partial t of 256 adds the squares of elements t,
// t + 256, ..., t + 1792 in that order; the partials fold by halving, partial[t] += partial[t + width],
// width = 128 .. 1.  With element 256 g + 8 l + j of the row in v[8 g + j] of lane l, a lane holds the
// eight elements of partials 8 l .. 8 l + 7: the halvings of width 128 .. 8 are the lane butterfly of
// each partial j, the last three are ((q0 + q4) + (q2 + q6)) + ((q1 + q5) + (q3 + q7)) -- the 16, 8, 4
// exchanges after warp_reduce8.  Every lane returns the total.
__device__ __forceinline__ float row_sumsq_2048(const float* v, int lane) {
  float part[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float acc = 0.0f;
#pragma unroll
    for (int g = 0; g < 8; ++g) acc = __fmaf_rn(v[8 * g + j], v[8 * g + j], acc);
    part[j] = acc;
  }
  float q = warp_reduce8(part, lane);       // q_j on the lanes with reduce8_slot(lane) == j
  q = __fadd_rn(q, __shfl_xor_sync(0xffffffffu, q, 16));   // j ^ 4
  q = __fadd_rn(q, __shfl_xor_sync(0xffffffffu, q, 8));    // j ^ 2
  q = __fadd_rn(q, __shfl_xor_sync(0xffffffffu, q, 4));    // j ^ 1
  return q;
}

// acc += x[0..7] * w[0..7]; w is one 16-byte vector of 8 BF16 values.
__device__ __forceinline__ float fma8(const float* x, const uint4& w, float acc) {
  acc = __fmaf_rn(x[0], bf16_lo(w.x), acc);
  acc = __fmaf_rn(x[1], bf16_hi(w.x), acc);
  acc = __fmaf_rn(x[2], bf16_lo(w.y), acc);
  acc = __fmaf_rn(x[3], bf16_hi(w.y), acc);
  acc = __fmaf_rn(x[4], bf16_lo(w.z), acc);
  acc = __fmaf_rn(x[5], bf16_hi(w.z), acc);
  acc = __fmaf_rn(x[6], bf16_lo(w.w), acc);
  acc = __fmaf_rn(x[7], bf16_hi(w.w), acc);
  return acc;
}

__device__ __forceinline__ void unpack8(const uint4& v, float* out) {
  out[0] = bf16_lo(v.x); out[1] = bf16_hi(v.x);
  out[2] = bf16_lo(v.y); out[3] = bf16_hi(v.y);
  out[4] = bf16_lo(v.z); out[5] = bf16_hi(v.z);
  out[6] = bf16_lo(v.w); out[7] = bf16_hi(v.w);
}

// ---------------------------------------------------------------------------
// Timers and memory-ordering primitives
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(
    const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_s32(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_cg_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_cg_f32(const void* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint16_t ld_cg_u16(const void* p) {
  uint16_t v;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
  return v;
}

// ---------------------------------------------------------------------------
// Shared-memory mbarriers and 1-D bulk (TMA) copies
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
               :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// global -> shared bulk copy; bytes % 16 == 0, both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src,
                                         uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1], %2, [%3];"
      :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(p), "r"(bytes) : "memory");
}

// Bounded wait on an mbarrier phase.  Returns false when the budget ran out or
// another thread of the block already raised `abort_flag`.  `diag` (may be
// nullptr) receives {spins, elapsed ns lo, barrier word lo, barrier word hi}
// when this call is the one that ran out of budget.
static __device__ __noinline__ bool mbar_wait_bounded_slow(uint32_t bar, uint32_t parity,
                                                    volatile int* abort_flag, unsigned* diag) {
  const unsigned long long start = global_timer_ns();
  unsigned spins = 0;
  while (!mbar_test(bar, parity)) {
    if ((++spins & 255u) == 0u) {
      if (*abort_flag != 0) return false;
      const unsigned long long elapsed = global_timer_ns() - start;
      if (elapsed > kWaitBudgetNs) {
        *abort_flag = kStatusTimeoutMbarrier;
        if (diag != nullptr) {
          unsigned lo, hi;
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(bar) : "memory");
          diag[0] = spins;
          diag[1] = static_cast<unsigned>(elapsed >> 10);
          diag[2] = lo;
          diag[3] = hi;
        }
        return false;
      }
    }
  }
  return true;
}
// The common case -- the phase has completed, or completes within a few probes -- stays inline; the
// timed loop is one shared out-of-line function, which keeps the persistent kernels' text small
// (their per-layer code runs once per layer, so every kilobyte of it is an instruction-cache miss).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int* abort_flag,
                                                  unsigned* diag = nullptr) {
#pragma unroll 1
  for (int probe = 0; probe < 4; ++probe) {
    if (mbar_test(bar, parity)) return true;
  }
  return mbar_wait_bounded_slow(bar, parity, abort_flag, diag);
}

// Programmatic dependent launch.  A kernel launched with launch_pdl may have its blocks placed
// while the kernel before it in the stream is still running; it must call pdl_enter() before its
// first access to global memory: that waits until the predecessor has completed and its writes are
// visible (a no-op for a kernel launched the ordinary way), after telling the scheduler that the
// kernel after this one may be placed early as well.
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Whether launch_pdl relaxes the serialisation is the calling thread's choice for the span of one
// host call (PdlScope): overlapping the kernel boundaries gains 3-4 % on a prefill layer of up to
// 2048 tokens, where the gaps between its ten kernels weigh most, and loses 2-3 % at 4096 and 8192
// tokens, so the prefill entry points relax it only up to pdl_max_tokens().
inline thread_local bool t_pdl_relaxed = true;
struct PdlScope {
  bool saved;
  explicit PdlScope(bool relaxed) : saved(t_pdl_relaxed) { t_pdl_relaxed = relaxed; }
  ~PdlScope() { t_pdl_relaxed = saved; }
  PdlScope(const PdlScope&) = delete;
  PdlScope& operator=(const PdlScope&) = delete;
};
// AIMA_MOE_PDL_MAX_TOKENS in the environment moves the limit (0: plain stream order everywhere).
inline int pdl_max_tokens() {
  static const int limit = [] {
    const char* v = std::getenv("AIMA_MOE_PDL_MAX_TOKENS");
    return (v != nullptr && v[0] != '\0') ? std::atoi(v) : 2048;
  }();
  return limit;
}


// Opt-in of one kernel to more than 48 KB of dynamic shared memory.  The attribute belongs to the
// (function, device) pair, so it is set once per device the calling thread has made current -- a
// process may drive several GPUs -- under a mutex, because several host threads may launch at once.
template <auto Kernel>
inline cudaError_t opt_in_dynamic_smem(int bytes) {
  static std::mutex mutex;
  static unsigned long long done[4] = {0, 0, 0, 0};      // one bit per device ordinal
  int device = -1;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return error;
  std::lock_guard<std::mutex> lock(mutex);
  const bool tracked = device >= 0 && device < 256;
  if (tracked && ((done[device >> 6] >> (device & 63)) & 1ull) != 0ull) return cudaSuccess;
  error = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (error == cudaSuccess && tracked) done[device >> 6] |= 1ull << (device & 63);
  return error;
}

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem_bytes,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = t_pdl_relaxed ? 1 : 0;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

}  // namespace aima
