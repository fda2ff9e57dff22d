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
//   --- grid barrier: all 256 logits known -> top-8 (warp 0 of every block)
//   1   routed gate/up rows of the 8 chosen experts (8 KB "pair" items through
//       a 10-slot ring); meanwhile the block's slice of the down projection
//       (8 experts + shared, <= 126 KB) is already being copied into a second
//       shared-memory region
//   --- grid barrier: all SwiGLU activations known
//   2   down products for the block's <= 14 output elements, weighted sum,
//       shared expert, residual add, store
//   --- grid barrier: next layer's input complete
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
constexpr int kOffDots = kOffAct + kDownRegionRanks * kInter * 2;                  // +9216
constexpr int kOffMisc = kOffDots + kDecodeMaxRowsPerBlock * kDotsStride * 4;      // +672
constexpr int kMiscBytes = 512;
constexpr int kOffBars = kOffMisc + kMiscBytes;
constexpr int kBarCount = 2 * kRingSlots + 1;
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
  Misc* misc = reinterpret_cast<Misc*>(smem + kOffMisc);
  const uint32_t bars = smem_u32(smem + kOffBars);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kRingSlots + s); };
  const uint32_t down_bar = bars + 8u * (2 * kRingSlots);

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

  if (warp == kDecodeConsumerWarps) {
    // ------------------------------ producer ------------------------------
    unsigned seq = 0;
    unsigned issued[kRingSlots];
#pragma unroll
    for (int s = 0; s < kRingSlots; ++s) issued[s] = 0;
    unsigned down_issued = 0;
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
        const int burst = min(p1 - p0, kRingSlots - 2);
        auto issue_down = [&]() {
          const uint32_t rank_bytes = nh * kDownRowBytes;
          mbar_arrive_expect_tx(down_bar, rank_bytes * (n_local + 1));
          for (int q = 0; q < n_local; ++q) {
            const int e_local = misc->ids[misc->local_rank[q]] - p.expert_lo;
            const __nv_bfloat16* src = L.expert_down +
                (static_cast<size_t>(e_local) * kHidden + h0) * kInter;
            bulk_g2s(smem_u32(down_region + q * kDecodeMaxRowsPerBlock * kDownRowBytes),
                     src, rank_bytes, down_bar);
          }
          bulk_g2s(smem_u32(down_region + kTopK * kDecodeMaxRowsPerBlock * kDownRowBytes),
                   L.shared_down_proj + static_cast<size_t>(h0) * kInter, rank_bytes, down_bar);
          down_issued = li + 1;
        };
        for (int pi = p0; pi < p1 && alive; ++pi) {
          if (pi - p0 == burst) issue_down();
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
        if (!alive) break;
        if (p1 - p0 <= burst) issue_down();
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
      const LayerPtrs L = p.layers[p.first_layer + li];
      const __nv_bfloat16* x_src = first ? p.x_in : ((li & 1) ? p.xbuf1 : p.xbuf0);
      __nv_bfloat16* x_dst = last ? p.x_out : ((li & 1) ? p.xbuf0 : p.xbuf1);

      stamp(li, 0);
      // ---- norm: h2 in registers, element k = 256 g + 8 lane + j at xr[8 g + j]
      float xr[64];
      {
        float total = 0.0f;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint4 v = ld_cg_u4(reinterpret_cast<const uint4*>(x_src) + g * 32 + lane);
          unpack8(v, xr + 8 * g);
          float part = 0.0f;
#pragma unroll
          for (int j = 0; j < 8; ++j) part = __fmaf_rn(xr[8 * g + j], xr[8 * g + j], part);
          part = butterfly_sum(part);
          total = (g == 0) ? part : __fadd_rn(total, part);
        }
        const float inv = det_rsqrtf(__fadd_rn(__fdiv_rn(total, static_cast<float>(kHidden)), p.eps));
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint4 wv = __ldg(reinterpret_cast<const uint4*>(L.norm_weight) + g * 32 + lane);
          float wf[8];
          unpack8(wv, wf);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float scaled = __fmul_rn(xr[8 * g + j], inv);
            xr[8 * g + j] = round_bf16(__fmul_rn(scaled, __fadd_rn(wf[j], 1.0f)));
          }
        }
        if (p.dbg_h2 != nullptr && c == 0 && warp == 0) {
#pragma unroll
          for (int g = 0; g < 8; ++g)
#pragma unroll
            for (int j = 0; j < 8; ++j)
              p.dbg_h2[256 * g + 8 * lane + j] = __float2bfloat16_rn(xr[8 * g + j]);
        }
      }

      stamp(li, 1);
      // ---- R items ----
      const int n_r_items = 1 + n_shared_pairs + (owns_gate_row ? 1 : 0);
      for (int k = 0; k < n_r_items && alive; ++k) {
        const unsigned item = seq + k;
        if (static_cast<int>(item % kRingSlots) != warp) continue;
        const uint8_t* slot = wait_item(item, 2);
        if (slot == nullptr) { alive = false; break; }
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
            p.logits[c] = v0;
            if (eb < kExperts) p.logits[eb] = v1;
          } else if (k <= n_shared_pairs) {
            const int i = c + (k - 1) * G;
            const float g = round_bf16(a);
            const float u = round_bf16(b);
            p.act[kTopK * kInter + i] = float_to_bf16_bits(__fmul_rn(det_silu(g), u));
          } else {
            *p.gate_logit = round_bf16(a);
          }
        }
      }
      seq += n_r_items;
      stamp(li, 2);
      // (an aborted warp still joins the barriers below; they return false)
      if (!grid_barrier(p, bar_base + (++nbar) * G, abort_flag, decision, ctid)) break;
      stamp(li, 3);

      // ---- top-8, ties to the lowest expert id; softmax over the eight ----
      if (warp == 0) {
        float v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = ld_cg_f32(p.logits + 32 * q + lane);
        if (p.dbg_logits != nullptr && c == 0) {
#pragma unroll
          for (int q = 0; q < 8; ++q) p.dbg_logits[32 * q + lane] = v[q];
        }
        float sel_v[kTopK];
        int sel_i[kTopK];
#pragma unroll
        for (int r = 0; r < kTopK; ++r) {
          float best = v[0];
          int best_id = lane;
#pragma unroll
          for (int q = 1; q < 8; ++q) {
            if (v[q] > best) { best = v[q]; best_id = 32 * q + lane; }
          }
#pragma unroll
          for (int s = 16; s >= 1; s >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, s);
            const int oi = __shfl_xor_sync(0xffffffffu, best_id, s);
            if (ov > best || (ov == best && oi < best_id)) { best = ov; best_id = oi; }
          }
          sel_v[r] = best;
          sel_i[r] = best_id;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (best_id == 32 * q + lane) v[q] = -CUDART_INF_F;
          }
        }
        float ex[kTopK];
        float denom = 0.0f;
#pragma unroll
        for (int r = 0; r < kTopK; ++r) {
          ex[r] = det_expf(__fsub_rn(sel_v[r], sel_v[0]));
          denom = __fadd_rn(denom, ex[r]);
        }
        if (lane == 0) {
          int n_local = 0;
#pragma unroll
          for (int r = 0; r < kTopK; ++r) {
            const uint16_t wb = float_to_bf16_bits(__fdiv_rn(ex[r], denom));
            misc->ids[r] = sel_i[r];
            misc->weights[r] = bf16_bits_to_float(wb);
            if (sel_i[r] >= p.expert_lo && sel_i[r] < p.expert_hi) misc->local_rank[n_local++] = r;
            if (c == 0) {
              if (p.dbg_ids != nullptr) p.dbg_ids[r] = sel_i[r];
              if (p.dbg_scores != nullptr) p.dbg_scores[r] = sel_v[r];
              if (p.dbg_weights != nullptr) reinterpret_cast<uint16_t*>(p.dbg_weights)[r] = wb;
            }
          }
          misc->n_local = n_local;
          __threadfence_block();
          misc->ids_layer = li + 1;
        }
      }
      consumer_sync();
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
        if (slot == nullptr) { alive = false; break; }
        float a, b;
        pair_dot(slot, xr, a, b);
        release_item(item);
        if (lane == 0) p.act[pi] = float_to_bf16_bits(__fmul_rn(det_silu(a), b));
      }
      seq += (p1 - p0);
      stamp(li, 5);
      if (!grid_barrier(p, bar_base + (++nbar) * G, abort_flag, decision, ctid)) break;
      stamp(li, 6);

      // ---- phase 2: down products for outputs h0 .. h1-1 ----
      for (int v = ctid; v < kDownRegionRanks * kInter * 2 / 16; v += kDecodeConsumerThreads) {
        reinterpret_cast<uint4*>(act_s)[v] = ld_cg_u4(reinterpret_cast<const uint4*>(p.act) + v);
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
      stamp(li, 8);
      if (alive) {
        const int per_row = n_local + 1;
        const int n_dots = nh * per_row;
        for (int d = warp; d < n_dots; d += kDecodeConsumerWarps) {
          const int hh = d / per_row;
          const int q = d - hh * per_row;
          const int region = (q == n_local) ? kTopK : q;
          const uint4* wrow = reinterpret_cast<const uint4*>(
              down_region + (region * kDecodeMaxRowsPerBlock + hh) * kDownRowBytes) + lane;
          const uint4* arow = reinterpret_cast<const uint4*>(act_s + region * kInter) + lane;
          float acc = 0.0f;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            float af[8];
            unpack8(arow[i * 32], af);
            acc = fma8(af, wrow[i * 32], acc);
          }
          acc = butterfly_sum(acc);
          if (lane == 0) dots[hh * kDotsStride + region] = acc;
        }
      }
      if (!uniform_alive(abort_flag, decision, ctid)) break;
      stamp(li, 9);
      if (ctid < nh) {
        const int h = h0 + ctid;
        float acc = 0.0f;
        for (int q = 0; q < n_local; ++q) {
          acc = __fmaf_rn(misc->weights[misc->local_rank[q]], dots[ctid * kDotsStride + q], acc);
        }
        const float routed = round_bf16(acc);
        const float sig = round_bf16(det_sigmoid(ld_cg_f32(p.gate_logit)));
        const float shared_down = round_bf16(dots[ctid * kDotsStride + kTopK]);
        const float shared_scaled = round_bf16(__fmul_rn(sig, shared_down));
        const float combined = round_bf16(__fadd_rn(routed, shared_scaled));
        const float resid = bf16_bits_to_float(ld_cg_u16(reinterpret_cast<const uint16_t*>(x_src) + h));
        x_dst[h] = __float2bfloat16_rn(__fadd_rn(resid, combined));
        if (p.dbg_routed != nullptr) p.dbg_routed[h] = __float2bfloat16_rn(routed);
        if (p.dbg_shared_scaled != nullptr) p.dbg_shared_scaled[h] = __float2bfloat16_rn(shared_scaled);
      }
      stamp(li, 10);
      if (!last) {
        if (!grid_barrier(p, bar_base + (++nbar) * G, abort_flag, decision, ctid)) break;
      }
      stamp(li, 11);
    }
    if (c == 0 && ctid == 0 && *abort_flag == 0) {
      *p.bar_base = bar_base + nbar * G;
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
