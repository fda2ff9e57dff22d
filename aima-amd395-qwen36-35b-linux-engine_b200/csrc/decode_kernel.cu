// Batch-1 decode of the MoE half-layer as ONE persistent cooperative kernel.
//
// Replaces, per layer, the ten launches of the reference decode path
// (native/src/native_linear_layer.hip.cpp:163-187): RMSNorm, the fused
// 1025-wide shared projection, shared SiLU*up, shared down GEMV, sigmoid scale,
// router stage 1 / stage 2, routed gate_up + SiLU, routed down + weighted sum
// and the final add pair; arithmetic follows
// benchmarks/shape-lab/four_layer_mini_engine.py:304-326, 391-473, 844-859,
// 1152-1220 and native/src/native_pointwise.hip.cpp:94-107, 184-205.
//
// Structure.  One block per SM.  Warp 15 is a producer that streams weight rows
// from HBM into shared memory with 1-D bulk (TMA) copies; warps 0-14 consume
// them with the canonical warp dot product.  The kernel is bandwidth bound
// (57.7 MB of weights per layer for ~30 MFLOP), so everything is arranged to
// keep bulk copies in flight across the three grid-wide synchronisations a
// layer needs:
//
//   R   every block: norm of the 2048-vector (per warp, registers), its share
//       of the 256 router rows and of the 513 shared-expert input pairs
//   --- logits exchange: every logit travels as one 64-bit word {tag, value};
//       warp 0 of every block polls the 256 words, then takes the top-8
//   1   routed gate/up rows of the 8 chosen experts (8 KB "pair" items through
//       a 10-slot ring); meanwhile the block's slice of the down projection
//       (8 experts + shared, <= 126 KB) is already being copied into a second
//       shared-memory region
//   --- grid barrier: all SwiGLU activations known
//   2   down products for the block's <= 14 output elements, weighted sum,
//       shared expert, residual add, store
//   --- output exchange: the 2048 outputs travel as 32-bit words {tag, bf16};
//       four warps of every block poll them into shared memory
// Data that carries its own tag needs no separate barrier and no second round
// trip through L2; only the activation hand-over is a counter barrier, and it
// hides behind the arrival of the down-projection rows.
//
// Every wait (mbarrier, grid barrier, hand-over of the expert ids to the
// producer) is bounded; on expiry the block raises a status word, drains its
// outstanding copies and returns, so the context stays usable.
#include "decode_kernel.cuh"

#include <math_constants.h>

namespace aima {
namespace {

// Ring of weight "pair" slots.  Item i always lands in slot i % kRingSlots and is
// always consumed by warp i % kRingSlots: a parity wait on an mbarrier is only
// meaningful when the waiter is at most one phase behind, so consecutive uses
// of a slot must be consumed in order by one warp.  Warps kRingSlots..14 only
// take part in the top-8 and down-projection phases.
constexpr int kRingSlots = 10;
constexpr int kSlotBytes = 8192;               // two 4 KB weight rows
constexpr int kRowBytes = kHidden * 2;         // 4096
constexpr int kDownRowBytes = kInter * 2;      // 1024
constexpr int kDownRegionRanks = kTopK + 1;    // 8 routed + shared
constexpr int kDotsStride = 12;

// shared-memory map (bytes)
constexpr int kOffRing = 0;
constexpr int kOffDown = kOffRing + kRingSlots * kSlotBytes;                       // 81920
constexpr int kOffAct = kOffDown + kDownRegionRanks * kDecodeMaxRowsPerBlock * kDownRowBytes;  // +129024
constexpr int kActBytes = kDownRegionRanks * kInter * 2 + 16;                      // 9 x 512 BF16 + gate logit
constexpr int kOffDots = kOffAct + kActBytes;                                      // +9232
constexpr int kOffX = kOffDots + kDecodeMaxRowsPerBlock * kDotsStride * 4;         // +672: layer input, packed BF16
constexpr int kOffNorm = kOffX + kHidden * 2;                                      // +4096: norm weight row
constexpr int kOffMisc = kOffNorm + kHidden * 2;                                   // +4096
constexpr int kMiscBytes = 512;
constexpr int kOffBars = kOffMisc + kMiscBytes;
constexpr int kBarCount = 2 * kRingSlots + 2;
constexpr int kSmemTotal = kOffBars + kBarCount * 8;
static_assert(kSmemTotal <= 227 * 1024, "decode kernel shared memory exceeds 227 KB");
static_assert(kSmemTotal == kDecodeSmemBytes, "keep decode_kernel.cuh in step");

struct Misc {
  int ids[kTopK];          // selected experts in selection order
  float weights[kTopK];    // BF16-rounded routing weights as FP32
  int local_rank[kTopK];   // ranks r whose expert lives on this GPU, ascending
  int n_local;
  volatile int ids_layer;  // (layer ordinal + 1) the ids above belong to
  volatile int abort_flag; // block-local copy of a raised status
  volatile int decision;   // block-uniform "keep going" verdict (see uniform_alive)
};
static_assert(sizeof(Misc) <= kMiscBytes, "Misc too large");
static_assert(kRingSlots <= kDecodeConsumerWarps, "each ring slot needs its own consumer warp");

__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" :: "n"(kDecodeConsumerThreads) : "memory");
}

__device__ __forceinline__ void raise_status(const DecodeParams& p,
                                             volatile int* abort_flag, int code) {
  atomicCAS(p.status, 0, code);
  *abort_flag = code;
}

// Records where the first bounded wait gave up: status[1] = site, [2] = block,
// [3] = warp, [4] = item / layer detail.  Sites: 1 producer slot acquire,
// 2 consumer item (router / shared rows), 3 consumer item (routed rows),
// 4 down-projection region, 5 grid barrier, 6 expert-id hand-over.
__device__ __forceinline__ void record_site(const DecodeParams& p, int site, int detail,
                                            const unsigned* diag = nullptr) {
  if (atomicCAS(p.status + 1, 0, site) == 0) {
    p.status[2] = blockIdx.x;
    p.status[3] = threadIdx.x >> 5;
    p.status[4] = detail;
    if (diag != nullptr) {
      p.status[5] = static_cast<int>(diag[0]);
      p.status[6] = static_cast<int>(diag[1]);
      p.status[7] = static_cast<int>(diag[2]);
      p.status[8] = static_cast<int>(diag[3]);
    }
  }
}

// Grid-wide barrier over the consumer threads of all blocks.
__device__ __forceinline__ bool grid_barrier(const DecodeParams& p,
                                             unsigned long long target,
                                             volatile int* abort_flag,
                                             volatile int* decision, int ctid) {
  consumer_sync();
  if (ctid == 0 && *abort_flag == 0) {
    __threadfence();
    atomicAdd(p.bar_counter, 1ull);
    const unsigned long long start = global_timer_ns();
    unsigned spins = 0;
    while (ld_acquire_u64(p.bar_counter) < target) {
      if ((++spins & 63u) == 0u) {
        const int remote = ld_relaxed_s32(p.status);
        if (remote != 0) { *abort_flag = remote; break; }
        if (global_timer_ns() - start > kWaitBudgetNs) {
          raise_status(p, abort_flag, kStatusTimeoutGridBarrier);
          record_site(p, 5, static_cast<int>(target));
          break;
        }
      }
    }
  }
  if (ctid == 0) *decision = (*abort_flag == 0) ? 1 : 0;
  consumer_sync();
  return *decision != 0;
}

// Block-uniform verdict on whether any thread of the block has raised a status.
// abort_flag can be set at any moment (e.g. by the producer warp), so consumer
// threads must not branch on it directly around a named barrier: thread 0
// samples it once and everybody follows that sample.
__device__ __forceinline__ bool uniform_alive(volatile int* abort_flag,
                                              volatile int* decision, int ctid) {
  consumer_sync();
  if (ctid == 0) *decision = (*abort_flag == 0) ? 1 : 0;
  consumer_sync();
  return *decision != 0;
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
__device__ __forceinline__ int reduce8_lane(int d) {
  return ((d >> 2) & 1) * 16 + ((d >> 1) & 1) * 8 + (d & 1) * 4;
}

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Exchange words are polled while other blocks are still writing them, so both
// sides use STRONG (relaxed, gpu-scope) accesses: a weak ld.global.cg may keep
// being served a snapshot of the line taken on the poller's side of the chip.
__device__ __forceinline__ unsigned long long ld_strong_u64(const void* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_strong_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_strong_u64(void* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}
// system scope: the other end is another GPU reached over NVLink
__device__ __forceinline__ unsigned long long ld_sys_u64(const void* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_u64(void* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_strong_u32(void* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

// Number of shared-expert input pairs block c owns: i = c, c+G, ... < 512.
__device__ __forceinline__ int shared_pairs_of(int c, int G) {
  return c < kSharedInter ? (kSharedInter - 1 - c) / G + 1 : 0;
}

}  // namespace

__global__ void __launch_bounds__(kDecodeThreads, 1)
moe_decode_persistent_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem + kOffRing;
  uint8_t* down_region = smem + kOffDown;
  uint16_t* act_s = reinterpret_cast<uint16_t*>(smem + kOffAct);
  float* dots = reinterpret_cast<float*>(smem + kOffDots);
  uint8_t* x_s = smem + kOffX;
  uint8_t* norm_s = smem + kOffNorm;
  Misc* misc = reinterpret_cast<Misc*>(smem + kOffMisc);
  const uint32_t bars = smem_u32(smem + kOffBars);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kRingSlots + s); };
  const uint32_t down_bar = bars + 8u * (2 * kRingSlots);
  const uint32_t norm_bar = bars + 8u * (2 * kRingSlots + 1);

  const int G = gridDim.x;
  const int c = blockIdx.x;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &misc->abort_flag;
  volatile int* decision = &misc->decision;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRingSlots; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(down_bar, 1);
    mbar_init(norm_bar, 1);
    // every ring slot starts out released: complete phase 0 of its empty barrier
    for (int s = 0; s < kRingSlots; ++s) mbar_arrive(empty_bar(s));
    misc->ids_layer = 0;
    misc->abort_flag = 0;
    misc->decision = 1;
    misc->n_local = 0;
    mbar_fence_init();
  }
  __syncthreads();

  const int h0 = (c * kHidden) / G;
  const int h1 = ((c + 1) * kHidden) / G;
  const int nh = h1 - h0;
  const int eb = c + G;                       // second router row of this block
  const int n_shared_pairs = shared_pairs_of(c, G);
  const bool owns_gate_row = (c == G - 1);
  const unsigned long long bar_base = *p.bar_base;
  const unsigned epoch0 = *p.epoch_base;      // exchange tag of layer ordinal li is epoch0 + li + 1

  if (warp == kDecodeConsumerWarps) {
    // ------------------------------ producer ------------------------------
    unsigned seq = 0;
    unsigned issued[kRingSlots];
#pragma unroll
    for (int s = 0; s < kRingSlots; ++s) issued[s] = 0;
    unsigned down_issued = 0;
    unsigned norm_issued = 0;
    bool alive = true;

    // acquire a ring slot for item `seq`; returns slot index or -1
    auto acquire = [&](unsigned item) -> int {
      const int s = item % kRingSlots;
      const unsigned use = item / kRingSlots;
      unsigned diag[4] = {0, 0, 0, 0};
      if (!mbar_wait_bounded(empty_bar(s), use & 1u, abort_flag, diag)) {
        if (*abort_flag == kStatusTimeoutMbarrier) {
          atomicCAS(p.status, 0, kStatusTimeoutMbarrier);
          record_site(p, 1, static_cast<int>(item), diag);
        }
        return -1;
      }
      return s;
    };

    if (lane == 0) {
      for (int li = 0; li < p.n_layers && alive; ++li) {
        const LayerPtrs L = p.layers[p.first_layer + li];
        // ---- norm weight row into its own region (its readers finished before the ids of the
        //      previous layer were published, which this thread has waited for) ----
        mbar_arrive_expect_tx(norm_bar, kRowBytes);
        bulk_g2s(smem_u32(norm_s), L.norm_weight, kRowBytes, norm_bar);
        norm_issued = li + 1;
        // ---- R items: router rows, shared input pairs, shared gate row ----
        {
          const int s = acquire(seq);
          if (s < 0) { alive = false; break; }
          const uint32_t dst = smem_u32(ring + s * kSlotBytes);
          const uint32_t bytes = kRowBytes * (eb < kExperts ? 2 : 1);
          mbar_arrive_expect_tx(full_bar(s), bytes);
          bulk_g2s(dst, L.router + static_cast<size_t>(c) * kHidden, kRowBytes, full_bar(s));
          if (eb < kExperts)
            bulk_g2s(dst + kRowBytes, L.router + static_cast<size_t>(eb) * kHidden, kRowBytes, full_bar(s));
          issued[s] = seq / kRingSlots + 1;
          ++seq;
        }
        for (int k = 0; k < n_shared_pairs && alive; ++k) {
          const int i = c + k * G;
          const int s = acquire(seq);
          if (s < 0) { alive = false; break; }
          const uint32_t dst = smem_u32(ring + s * kSlotBytes);
          mbar_arrive_expect_tx(full_bar(s), 2 * kRowBytes);
          bulk_g2s(dst, L.shared_gate_proj + static_cast<size_t>(i) * kHidden, kRowBytes, full_bar(s));
          bulk_g2s(dst + kRowBytes, L.shared_up_proj + static_cast<size_t>(i) * kHidden, kRowBytes, full_bar(s));
          issued[s] = seq / kRingSlots + 1;
          ++seq;
        }
        if (!alive) break;
        if (owns_gate_row) {
          const int s = acquire(seq);
          if (s < 0) { alive = false; break; }
          const uint32_t dst = smem_u32(ring + s * kSlotBytes);
          mbar_arrive_expect_tx(full_bar(s), kRowBytes);
          bulk_g2s(dst, L.shared_gate, kRowBytes, full_bar(s));
          issued[s] = seq / kRingSlots + 1;
          ++seq;
        }
        // ---- wait for this layer's expert ids ----
        {
          const unsigned long long start = global_timer_ns();
          unsigned spins = 0;
          while (misc->ids_layer != li + 1) {
            if ((++spins & 255u) == 0u) {
              if (*abort_flag != 0) { alive = false; break; }
              if (global_timer_ns() - start > kWaitBudgetNs) {
                raise_status(p, abort_flag, kStatusTimeoutIds);
                record_site(p, 6, li);
                alive = false;
                break;
              }
            }
          }
          if (!alive) break;
          __threadfence_block();
        }
        const int n_local = misc->n_local;
        const int n_pairs = n_local * kInter;
        const int p0 = static_cast<int>((static_cast<long long>(c) * n_pairs) / G);
        const int p1 = static_cast<int>((static_cast<long long>(c + 1) * n_pairs) / G);
        // The block's slice of the down projection is needed only after the activation barrier.  The
        // shared expert's rows (known without the routing) go first; the routed experts' rows are
        // requested AFTER the last gate/up pair, so they arrive while the block waits at the barrier
        // for the slowest block -- time in which HBM would otherwise idle -- instead of lengthening
        // the gate/up stream (21.5 -> 20.7 us per layer; issuing them 6 or 12 items before the end
        // gave 21.6 / 21.4).
        const uint32_t rank_bytes = nh * kDownRowBytes;
        mbar_arrive_expect_tx(down_bar, rank_bytes * (n_local + 1));
        bulk_g2s(smem_u32(down_region + kTopK * kDecodeMaxRowsPerBlock * kDownRowBytes),
                 L.shared_down_proj + static_cast<size_t>(h0) * kInter, rank_bytes, down_bar);
        down_issued = li + 1;
        for (int pi = p0; pi < p1 && alive; ++pi) {
          const int q = pi / kInter;
          const int i = pi - q * kInter;
          const int e_local = misc->ids[misc->local_rank[q]] - p.expert_lo;
          const int s = acquire(seq);
          if (s < 0) { alive = false; break; }
          const uint32_t dst = smem_u32(ring + s * kSlotBytes);
          const __nv_bfloat16* gate_row = L.expert_gate_up +
              (static_cast<size_t>(e_local) * (2 * kInter) + i) * kHidden;
          mbar_arrive_expect_tx(full_bar(s), 2 * kRowBytes);
          bulk_g2s(dst, gate_row, kRowBytes, full_bar(s));
          bulk_g2s(dst + kRowBytes, gate_row + static_cast<size_t>(kInter) * kHidden, kRowBytes, full_bar(s));
          issued[s] = seq / kRingSlots + 1;
          ++seq;
        }
        // also on the way out after a failed wait: the barrier's byte count must be met before the drain
        for (int q = 0; q < n_local; ++q) {
          const int e_local = misc->ids[misc->local_rank[q]] - p.expert_lo;
          const __nv_bfloat16* src = L.expert_down +
              (static_cast<size_t>(e_local) * kHidden + h0) * kInter;
          bulk_g2s(smem_u32(down_region + q * kDecodeMaxRowsPerBlock * kDownRowBytes),
                   src, rank_bytes, down_bar);
        }
        if (!alive) break;
      }
      // Drain: every copy this thread issued must have landed before the block
      // may exit (bounded; a phase that already completed returns at once).
      if (*abort_flag != 0) {
        for (int s = 0; s < kRingSlots; ++s) {
          if (issued[s] != 0) {
            volatile int ignore = 0;
            mbar_wait_bounded(full_bar(s), (issued[s] - 1u) & 1u, &ignore);
          }
        }
        if (down_issued != 0) {
          volatile int ignore = 0;
          mbar_wait_bounded(down_bar, (down_issued - 1u) & 1u, &ignore);
        }
        if (norm_issued != 0) {
          volatile int ignore = 0;
          mbar_wait_bounded(norm_bar, (norm_issued - 1u) & 1u, &ignore);
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ consumers -----------------------------
    const int ctid = threadIdx.x;                 // 0 .. 511
    unsigned seq = 0;                             // mirrors the producer's item counter
    unsigned long long nbar = 0;
    bool alive = true;

    // wait for item `item`, return slot pointer (nullptr on abort)
    auto wait_item = [&](unsigned item, int site) -> const uint8_t* {
      const int s = item % kRingSlots;
      const unsigned use = item / kRingSlots;
      unsigned diag[4] = {0, 0, 0, 0};
      if (!mbar_wait_bounded(full_bar(s), use & 1u, abort_flag, diag)) {
        if (*abort_flag == kStatusTimeoutMbarrier) {
          atomicCAS(p.status, 0, kStatusTimeoutMbarrier);
          record_site(p, site, static_cast<int>(item), diag);
        }
        return nullptr;
      }
      return ring + s * kSlotBytes;
    };
    auto release_item = [&](unsigned item) {
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(item % kRingSlots));
    };
    // two canonical 2048-dots of the register-resident vector against the two
    // rows of a slot
    auto pair_dot = [&](const uint8_t* slot, const float* xr, float& a, float& b) {
      a = 0.0f; b = 0.0f;
      const uint4* r0 = reinterpret_cast<const uint4*>(slot) + lane;
      const uint4* r1 = reinterpret_cast<const uint4*>(slot + kRowBytes) + lane;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 w0 = r0[i * 32];
        const uint4 w1 = r1[i * 32];
        a = fma8(xr + 8 * i, w0, a);
        b = fma8(xr + 8 * i, w1, b);
      }
      a = butterfly_sum(a);
      b = butterfly_sum(b);
    };

    // tracing stamps: 0 layer start, 1 norm done, 2 router/shared rows done, 3 logits barrier,
    // 4 top-8 done, 5 routed gate/up done, 6 activation barrier, 7 activations loaded,
    // 8 down region landed, 9 down dots done, 10 output stored, 11 output barrier
    auto stamp = [&](int li, int k) {
      if (p.timeline != nullptr && c == 0 && ctid == 0)
        p.timeline[li * kDecodeTraceStamps + k] = global_timer_ns();
    };
    for (int li = 0; li < p.n_layers; ++li) {
      const bool first = (li == 0);
      const bool last = (li == p.n_layers - 1);

      stamp(li, 0);
      const uint32_t* xw_src = (li & 1) ? p.xbuf1 : p.xbuf0;     // tagged words written by layer li - 1
      uint32_t* xw_dst = (li & 1) ? p.xbuf0 : p.xbuf1;
      const unsigned tag_in = (epoch0 + li) & 0xffffu;           // tag of layer li - 1
      const unsigned tag_out = (epoch0 + li + 1) & 0xffffu;
      // ---- layer input into shared memory (packed BF16) ----
      if (first) {
        if (ctid < kHidden / 8) {
          reinterpret_cast<uint4*>(x_s)[ctid] = ld_cg_u4(reinterpret_cast<const uint4*>(p.x_in) + ctid);
        }
      } else if (warp < 4) {
        // poll this warp's 512 tagged words until every tag is the previous layer's
        const uint4* src = reinterpret_cast<const uint4*>(xw_src + (c % kDecodeReplicas) * kHidden) + warp * 128 + lane;
        uint4 w[4];
        bool ready = false;
        const unsigned long long start = global_timer_ns();
        unsigned spins = 0;
        while (!ready) {
          bool mine = true;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            w[i] = ld_strong_u4(src + i * 32);
            mine = mine && (w[i].x >> 16) == tag_in && (w[i].y >> 16) == tag_in &&
                   (w[i].z >> 16) == tag_in && (w[i].w >> 16) == tag_in;
          }
          ready = __all_sync(0xffffffffu, mine);
          if (!ready && (++spins & 63u) == 0u) {
            if (*abort_flag != 0) break;
            if (global_timer_ns() - start > kWaitBudgetNs) {
              raise_status(p, abort_flag, kStatusTimeoutPeer);
              record_site(p, 7, li);
              break;
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint2 packed;
          packed.x = (w[i].x & 0xffffu) | (w[i].y << 16);
          packed.y = (w[i].z & 0xffffu) | (w[i].w << 16);
          reinterpret_cast<uint2*>(x_s)[warp * 128 + i * 32 + lane] = packed;
        }
      }
      if (!uniform_alive(abort_flag, decision, ctid)) break;
      // ---- norm, once per block: canonical sum of squares (warp g sums group g), then every
      //      thread normalises one 8-element chunk into h2_s (the activation region is idle now)
      uint8_t* h2_s = reinterpret_cast<uint8_t*>(act_s);
      if (warp < 8) {
        float xv[8];
        unpack8(reinterpret_cast<const uint4*>(x_s)[warp * 32 + lane], xv);
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = __fmaf_rn(xv[j], xv[j], acc);
        acc = butterfly_sum(acc);
        if (lane == 0) dots[warp] = acc;
      }
      consumer_sync();
      {
        float total = dots[0];
#pragma unroll
        for (int g = 1; g < 8; ++g) total = __fadd_rn(total, dots[g]);
        const float inv = det_rsqrtf(__fadd_rn(__fdiv_rn(total, static_cast<float>(kHidden)), p.eps));
        if (!mbar_wait_bounded(norm_bar, li & 1u, abort_flag)) {
          if (*abort_flag == kStatusTimeoutMbarrier) {
            atomicCAS(p.status, 0, kStatusTimeoutMbarrier);
            record_site(p, 8, li);
          }
          alive = false;
        }
        alive = __all_sync(0xffffffffu, alive);
        if (ctid < kHidden / 8) {
          float xv[8], wf[8];
          unpack8(reinterpret_cast<const uint4*>(x_s)[ctid], xv);
          unpack8(reinterpret_cast<const uint4*>(norm_s)[ctid], wf);
          uint32_t packed[4];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            const float a = __fmul_rn(__fmul_rn(xv[j], inv), __fadd_rn(wf[j], 1.0f));
            const float b = __fmul_rn(__fmul_rn(xv[j + 1], inv), __fadd_rn(wf[j + 1], 1.0f));
            packed[j / 2] = static_cast<uint32_t>(float_to_bf16_bits(a)) |
                            (static_cast<uint32_t>(float_to_bf16_bits(b)) << 16);
          }
          const uint4 out = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          reinterpret_cast<uint4*>(h2_s)[ctid] = out;
          if (p.dbg_h2 != nullptr && c == 0) reinterpret_cast<uint4*>(p.dbg_h2)[ctid] = out;
        }
      }
      consumer_sync();
      // streaming warps keep h2 in registers: element k = 256 g + 8 lane + j at xr[8 g + j]
      float xr[64];
      if (warp < kRingSlots) {
#pragma unroll
        for (int g = 0; g < 8; ++g) unpack8(reinterpret_cast<const uint4*>(h2_s)[g * 32 + lane], xr + 8 * g);
      }

      stamp(li, 1);
      // ---- R items ----
      const int n_r_items = 1 + n_shared_pairs + (owns_gate_row ? 1 : 0);
      for (int k = 0; k < n_r_items && alive; ++k) {
        const unsigned item = seq + k;
        if (static_cast<int>(item % kRingSlots) != warp) continue;
        const uint8_t* slot = wait_item(item, 2);
        if (!__all_sync(0xffffffffu, slot != nullptr)) { alive = false; break; }
        float a, b;
        pair_dot(slot, xr, a, b);
        release_item(item);
        if (lane == 0) {
          if (k == 0) {
            float v0 = a, v1 = b;
            if (p.router_bias != nullptr) {
              v0 = __fadd_rn(v0, p.router_bias[c]);
              if (eb < kExperts) v1 = __fadd_rn(v1, p.router_bias[eb]);
            }
            if (p.quant_eighths) {
              v0 = __fmul_rn(rintf(__fmul_rn(v0, 8.0f)), 0.125f);
              v1 = __fmul_rn(rintf(__fmul_rn(v1, 8.0f)), 0.125f);
            }
            const unsigned long long tag = static_cast<unsigned long long>(epoch0 + li + 1) << 32;
#pragma unroll
            for (int rep = 0; rep < kDecodeReplicas; ++rep) {
              st_strong_u64(p.logits + rep * kExperts + c, tag | __float_as_uint(v0));
              if (eb < kExperts) st_strong_u64(p.logits + rep * kExperts + eb, tag | __float_as_uint(v1));
            }
          } else if (k <= n_shared_pairs) {
            const int i = c + (k - 1) * G;
            const float g = round_bf16(a);
            const float u = round_bf16(b);
            const uint16_t bits = float_to_bf16_bits(__fmul_rn(det_silu(g), u));
#pragma unroll
            for (int rep = 0; rep < kDecodeReplicas; ++rep) p.act[rep * kDecodeActStride + kTopK * kInter + i] = bits;
          } else {
            const float gate = round_bf16(a);
#pragma unroll
            for (int rep = 0; rep < kDecodeReplicas; ++rep)
              *reinterpret_cast<float*>(p.act + rep * kDecodeActStride + 9 * kInter) = gate;
          }
        }
      }
      seq += n_r_items;
      stamp(li, 2);

      // ---- logits exchange + top-8 (ties to the lowest expert id) + softmax, warp 0 ----
      if (warp == 0) {
        const unsigned tag = epoch0 + li + 1;
        unsigned long long w[8];
        bool ready = false;
        const unsigned long long start = global_timer_ns();
        unsigned spins = 0;
        while (!ready) {
          bool mine = true;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            w[q] = ld_strong_u64(p.logits + (c % kDecodeReplicas) * kExperts + 32 * q + lane);
            mine = mine && static_cast<unsigned>(w[q] >> 32) == tag;
          }
          ready = __all_sync(0xffffffffu, mine);
          if (!ready && (++spins & 63u) == 0u) {
            if (*abort_flag != 0) break;
            if (global_timer_ns() - start > kWaitBudgetNs) {
              raise_status(p, abort_flag, kStatusTimeoutPeer);
              {
                // first expert whose word never carried this layer's tag, and what was there instead
                int bad = 0x7fffffff;
#pragma unroll
                for (int q = 7; q >= 0; --q)
                  if (static_cast<unsigned>(w[q] >> 32) != tag) bad = 32 * q + lane;
                const int first_bad = __reduce_min_sync(0xffffffffu, bad);
                int n_bad = 0;
#pragma unroll
                for (int q = 0; q < 8; ++q) n_bad += static_cast<unsigned>(w[q] >> 32) != tag ? 1 : 0;
                n_bad = __reduce_add_sync(0xffffffffu, n_bad);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  const unsigned m = __ballot_sync(0xffffffffu, static_cast<unsigned>(w[q] >> 32) != tag);
                  if (lane == 0 && p.status[1] == 0) p.status[16 + q] = static_cast<int>(m);
                }
                if (bad == first_bad) {
                  const unsigned long long word = w[(first_bad >> 5) & 7];
                  unsigned diag[4] = {tag, static_cast<unsigned>(first_bad),
                                      static_cast<unsigned>(n_bad) | (alive ? 0x10000u : 0u), static_cast<unsigned>(word >> 32)};
                  record_site(p, 9, li, diag);
                }
              }
              break;
            }
          }
        }
        stamp(li, 3);
        uint32_t k[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float value = __uint_as_float(static_cast<uint32_t>(w[q]));
          k[q] = order_key(value);
          if (p.dbg_logits != nullptr && c == 0) p.dbg_logits[32 * q + lane] = value;
        }
        float my_score = 0.0f;      // lane r keeps the r-th selected value
        int my_id = 0;
#pragma unroll 1
        for (int r = 0; r < kTopK; ++r) {
          uint32_t local = k[0];
#pragma unroll
          for (int q = 1; q < 8; ++q) local = max(local, k[q]);
          const uint32_t best = __reduce_max_sync(0xffffffffu, local);
          int candidate = 0x7fffffff;
#pragma unroll
          for (int q = 7; q >= 0; --q) {
            if (k[q] == best) candidate = 32 * q + lane;
          }
          const int winner = __reduce_min_sync(0xffffffffu, candidate);
          if (lane == r) { my_score = key_value(best); my_id = winner; }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (winner == 32 * q + lane) k[q] = 0u;
          }
        }
        // softmax over the eight: exp(s_r - s_0) / sum, summed in selection order
        const float top = __shfl_sync(0xffffffffu, my_score, 0);
        const float ex = det_expf(__fsub_rn(my_score, top));
        float denom = 0.0f;
#pragma unroll
        for (int r = 0; r < kTopK; ++r) denom = __fadd_rn(denom, __shfl_sync(0xffffffffu, ex, r));
        const uint16_t wb = float_to_bf16_bits(__fdiv_rn(ex, denom));
        const bool local_expert = my_id >= p.expert_lo && my_id < p.expert_hi;
        const unsigned local_mask = __ballot_sync(0xffffffffu, lane < kTopK && local_expert);
        if (lane < kTopK) {
          misc->ids[lane] = my_id;
          misc->weights[lane] = bf16_bits_to_float(wb);
          if (local_expert) misc->local_rank[__popc(local_mask & ((1u << lane) - 1u))] = lane;
          if (c == 0) {
            if (p.dbg_ids != nullptr) p.dbg_ids[lane] = my_id;
            if (p.dbg_scores != nullptr) p.dbg_scores[lane] = my_score;
            if (p.dbg_weights != nullptr) reinterpret_cast<uint16_t*>(p.dbg_weights)[lane] = wb;
          }
        }
        __syncwarp();
        if (lane == 0) {
          misc->n_local = __popc(local_mask);
          __threadfence_block();
          misc->ids_layer = li + 1;
        }
      }
      if (!uniform_alive(abort_flag, decision, ctid)) break;
      stamp(li, 4);

      // ---- phase 1: routed gate/up pairs of the experts held on this GPU ----
      const int n_local = misc->n_local;
      const int n_pairs = n_local * kInter;
      const int p0 = static_cast<int>((static_cast<long long>(c) * n_pairs) / G);
      const int p1 = static_cast<int>((static_cast<long long>(c + 1) * n_pairs) / G);
      for (int pi = p0; pi < p1 && alive; ++pi) {
        const unsigned item = seq + (pi - p0);
        if (static_cast<int>(item % kRingSlots) != warp) continue;
        const uint8_t* slot = wait_item(item, 3);
        if (!__all_sync(0xffffffffu, slot != nullptr)) { alive = false; break; }
        float a, b;
        pair_dot(slot, xr, a, b);
        release_item(item);
        if (lane == 0) {
          const uint16_t bits = float_to_bf16_bits(__fmul_rn(det_silu(a), b));
#pragma unroll
          for (int rep = 0; rep < kDecodeReplicas; ++rep) p.act[rep * kDecodeActStride + pi] = bits;
        }
      }
      seq += (p1 - p0);
      stamp(li, 5);
      if (!grid_barrier(p, bar_base + (++nbar) * G, abort_flag, decision, ctid)) break;
      stamp(li, 6);

      // ---- phase 2: down products for outputs h0 .. h1-1 ----
      for (int v = ctid; v < kActBytes / 16; v += kDecodeConsumerThreads) {
        reinterpret_cast<uint4*>(act_s)[v] = ld_cg_u4(
            reinterpret_cast<const uint4*>(p.act + (c % kDecodeReplicas) * kDecodeActStride) + v);
      }
      consumer_sync();
      stamp(li, 7);
      if (!mbar_wait_bounded(down_bar, li & 1u, abort_flag)) {
        if (*abort_flag == kStatusTimeoutMbarrier) {
          atomicCAS(p.status, 0, kStatusTimeoutMbarrier);
          record_site(p, 4, li);
        }
        alive = false;
      }
      alive = __all_sync(0xffffffffu, alive);
      stamp(li, 8);
      if (alive) {
        // unit = (rank slot q, half of the block's output rows): the activation row is unpacked
        // once and up to seven dots against it share one eight-way reduction
        const int half_rows = (nh + 1) / 2;
        const int n_units = 2 * (n_local + 1);
        for (int unit = warp; unit < n_units; unit += kDecodeConsumerWarps) {
          const int q = unit >> 1;
          const int row_base = (unit & 1) * half_rows;
          const int region = (q == n_local) ? kTopK : q;
          float af[16];
          {
            const uint4* arow = reinterpret_cast<const uint4*>(act_s + region * kInter) + lane;
            unpack8(arow[0], af);
            unpack8(arow[32], af + 8);
          }
          float part[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int hh = row_base + u;
            float acc = 0.0f;
            if (u < half_rows && hh < nh) {
              const uint4* wrow = reinterpret_cast<const uint4*>(
                  down_region + (region * kDecodeMaxRowsPerBlock + hh) * kDownRowBytes) + lane;
              acc = fma8(af, wrow[0], acc);
              acc = fma8(af + 8, wrow[32], acc);
            }
            part[u] = acc;
          }
          const float total = warp_reduce8(part, lane);
          const int u = reduce8_slot(lane);
          const int hh = row_base + u;
          if ((lane & 3) == 0 && u < half_rows && hh < nh) dots[hh * kDotsStride + region] = total;
        }
      }
      if (!uniform_alive(abort_flag, decision, ctid)) break;
      stamp(li, 9);
      // ---- expert parallelism: the down products of the rank slots held here go to every peer
      //      (plain stores over NVLink into its exchange buffer), those held elsewhere are polled
      //      from this GPU's own buffer; words carry the layer tag, buffers alternate per layer.
      //      Block c of every GPU owns the same output rows, so a peer can be at most one layer ahead.
      if (p.world > 1 && alive) {
        const unsigned long long tag64 = static_cast<unsigned long long>(epoch0 + li + 1) << 32;
        const size_t parity_base = static_cast<size_t>(li & 1) * kTopK * kHidden;
        const int sends = n_local * nh * (p.world - 1);
        for (int s = ctid; s < sends; s += kDecodeConsumerThreads) {
          const int peer_slot = s / (n_local * nh);
          const int rest = s - peer_slot * (n_local * nh);
          const int q = rest / nh;
          const int hh = rest - q * nh;
          const int peer = peer_slot + (peer_slot >= p.rank ? 1 : 0);
          const int slot = misc->local_rank[q];
          st_sys_u64(p.ep_dots[peer] + parity_base + static_cast<size_t>(slot) * kHidden + h0 + hh,
                     tag64 | __float_as_uint(dots[hh * kDotsStride + q]));
        }
      }
      if (ctid < nh) {
        const int h = h0 + ctid;
        float acc = 0.0f;
        if (p.world == 1) {
          for (int q = 0; q < n_local; ++q) {
            const float d = dots[ctid * kDotsStride + q];
            acc = __fmaf_rn(misc->weights[misc->local_rank[q]], d, acc);
            if (p.dbg_slot_dots != nullptr) p.dbg_slot_dots[misc->local_rank[q] * kHidden + h] = d;
          }
        } else {
          const unsigned tag = epoch0 + li + 1;
          const unsigned long long* mine = p.ep_dots[p.rank] + static_cast<size_t>(li & 1) * kTopK * kHidden + h;
          int q = 0;
          const unsigned long long start = global_timer_ns();
          for (int r = 0; r < kTopK; ++r) {
            float d;
            if (q < n_local && misc->local_rank[q] == r) {
              d = dots[ctid * kDotsStride + q];
              ++q;
            } else {
              unsigned long long word = ld_sys_u64(mine + static_cast<size_t>(r) * kHidden);
              unsigned spins = 0;
              while (static_cast<unsigned>(word >> 32) != tag) {
                if ((++spins & 63u) == 0u) {
                  if (*abort_flag != 0) break;
                  if (global_timer_ns() - start > kWaitBudgetNs) {
                    raise_status(p, abort_flag, kStatusTimeoutPeer);
                    record_site(p, 11, li * 16 + r);
                    break;
                  }
                }
                word = ld_sys_u64(mine + static_cast<size_t>(r) * kHidden);
              }
              d = __uint_as_float(static_cast<uint32_t>(word));
            }
            acc = __fmaf_rn(misc->weights[r], d, acc);
            if (p.dbg_slot_dots != nullptr) p.dbg_slot_dots[r * kHidden + h] = d;
          }
        }
        const float routed = round_bf16(acc);
        const float sig = round_bf16(det_sigmoid(*reinterpret_cast<const float*>(act_s + 9 * kInter)));
        const float shared_down = round_bf16(dots[ctid * kDotsStride + kTopK]);
        const float shared_scaled = round_bf16(__fmul_rn(sig, shared_down));
        const float combined = round_bf16(__fadd_rn(routed, shared_scaled));
        const float resid = bf16_bits_to_float(reinterpret_cast<const uint16_t*>(x_s)[h]);
        const uint16_t out_bits = float_to_bf16_bits(__fadd_rn(resid, combined));
        if (last) reinterpret_cast<uint16_t*>(p.x_out)[h] = out_bits;
        else {
#pragma unroll
          for (int rep = 0; rep < kDecodeReplicas; ++rep)
            st_strong_u32(xw_dst + rep * kHidden + h, (tag_out << 16) | out_bits);
        }
        if (p.dbg_routed != nullptr) p.dbg_routed[h] = __float2bfloat16_rn(routed);
        if (p.dbg_shared_scaled != nullptr) p.dbg_shared_scaled[h] = __float2bfloat16_rn(shared_scaled);
      }
      stamp(li, 10);
      stamp(li, 11);
    }
    if (c == 0 && ctid == 0 && *abort_flag == 0) {
      *p.bar_base = bar_base + nbar * G;
      *p.epoch_base = epoch0 + static_cast<unsigned>(p.n_layers);
    }
  }
  __syncthreads();
}

cudaError_t launch_moe_decode(const DecodeParams& params, int grid_blocks,
                              cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_decode_persistent_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kDecodeSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  DecodeParams local = params;
  void* args[] = {&local};
  return cudaLaunchCooperativeKernel(
      reinterpret_cast<const void*>(moe_decode_persistent_kernel), dim3(grid_blocks),
      dim3(kDecodeThreads), args, kDecodeSmemBytes, stream);
}

}  // namespace aima
