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
// Structure.  One block per SM, 16 warps.  Warp 4 is a producer that streams
// weights from HBM into ONE ring of 6 shared-memory slots of 32 KB (two halves
// of 16 KB) with 1-D bulk (TMA) copies; the twelve warps w with w % 4 != 0
// consume them with the canonical warp dot product, as three groups of four
// warps (slot s always belongs to group s % 3, its up to four rows or row pairs
// to the group's four warps); warp 0 runs the exchanges between blocks, the
// top-8 and the layer plan; warp 8 predicts the next layer's experts; warp 12
// is spare.  The kernel is bandwidth bound (57.7 MB of weights per layer for
// ~30 MFLOP) but its layer is a serial chain of three grid-wide hand-overs, so
// everything is arranged to keep bulk copies in flight across them.
//
// A bulk copy costs its issuing thread and the copy engine a fixed time whatever
// its size (one lane sustains about 8 copies of 4 KB per microsecond, 33 GB/s per
// SM, 4.9 TB/s over the chip: measured, and what an earlier version of this
// kernel that copied row by row was bound by), so every block is dealt
// CONTIGUOUS rows and fetches them 12-16 KB at a time, two lanes issuing.  Items
// of a layer pass through the ring in this order:
//
//   R1  router rows 2c, 2c+1 of this layer (half A) and the same two rows of the
//       NEXT layer's router (half B; prediction, see below); block 128 instead
//       carries the shared expert's gate row
//   R2  the block's 3-4 contiguous rows of the shared expert's gate (A) and up (B)
//       projections
//   B   "blind" items, requested with the experts PREDICTED for this layer while the previous
//       layer is still running: for each of the 8 expert positions the block's 3-4 contiguous
//       gate rows (A) and up rows (B).  The streaming warps turn them into activations as soon
//       as this layer's input is normalised, i.e. WHILE warp 0 is still waiting for the logits
//   --- logits exchange: every logit travels as one 64-bit word {tag, value};
//       warp 0 of every block polls the 256 words, takes the top-8, freezes the
//       blind issue and publishes the layer plan (which predicted positions hold
//       a chosen expert, which chosen experts still have to be fetched)
//   P   the gate/up chunks not covered by a valid blind item, with the real experts
//   D   the block's <= 14 rows of the down projections, two experts per item (shared expert first)
//   --- activation exchange: every SwiGLU activation travels as a 32-bit word {tag, bf16}; all warps
//       of every block poll the words of the used positions and of the shared expert into shared
//       memory (no barrier: the tags are the synchronisation); then
//       down products for the block's output elements from the down items,
//       weighted sum, shared expert, residual add
//   --- output exchange: the 2048 outputs travel as 32-bit words {tag, bf16};
//       eight warps of every block poll them into shared memory; after the RMSNorm the
//       normalised input stays in shared memory as FP32 and the dots read it from there
//
// Prediction.  A grid-wide hand-over through L2 costs about 1.5 us of pure latency
// (store, then a poll round trip), a layer has three of them, and nothing that
// depends on the routing can be requested before the second.  Applying the next
// layer's router to THIS layer's normalised input costs one more half item per
// block and predicts most of the next layer's experts.  Their rows are requested
// into the ring as slots fall free, their activations are computed before the
// routing is known, and a layer whose prediction was right has nothing left to
// fetch after its plan.  An activation computed blind is held back until the plan
// confirms its expert (a tagged word is final for its readers); a position whose
// prediction was wrong is fetched again with the right expert, so the result does
// not depend on the prediction: outputs are bit-identical with and without it.
//
// Every wait (mbarrier, exchange words, hand-overs between the warps of a block)
// is bounded; on expiry the block raises a status word, drains its outstanding
// copies and returns, so the context stays usable.
#include "decode_kernel.cuh"

#include <math_constants.h>

namespace aima {
namespace {

// Item i always lands in slot i % kRingSlots and is always consumed by warp group
// (i % kRingSlots) % kGroups: a parity wait on an mbarrier is only meaningful when
// the waiter is at most one phase behind, so consecutive uses of a slot must be
// consumed in order by the same warps.  Every warp of the group waits for and
// releases every item of its slots, whether it has a row of it or not.
constexpr int kRingSlots = 6;
constexpr int kGroups = 3;
constexpr int kGroupWarps = 4;
constexpr int kStreamWarps = kGroups * kGroupWarps;
// Warp roles.  An SM sub-partition issues for warps w, w + 4, w + 8, w + 12; warp 0 runs the serial part
// of every layer (polls, top-8, plan), so the other three warps of ITS sub-partition are the ones with
// little to issue (producer, predictor, spare) and the twelve streaming warps share the other three.
constexpr int kControlWarp = 0;
constexpr int kProducerWarp = 4;
constexpr int kPredictWarp = 8;
constexpr int kHalfBytes = 16384;              // <= 4 weight rows of 4 KB, or <= 14 down rows of 1 KB
constexpr int kSlotBytes = 2 * kHalfBytes;
constexpr int kRowBytes = kHidden * 2;         // 4096
constexpr int kDownRowBytes = kInter * 2;      // 1024
constexpr int kDotsStride = 12;
constexpr int kPositions = kTopK;              // ring positions a layer's experts are dealt to
constexpr int kRouterBlocks = kExperts / 2;    // blocks 0 .. 127 hold two router rows each, block 128 the shared gate row
// Blind tickets of a layer: ticket q is the gate/up chunk of position q.  (Down rows are not requested
// blind: they would sit in the ring until after the activation exchange, and a chunk that has to be
// fetched again after the plan could then find its slot taken by an item that cannot be consumed
// before it -- a cycle.  They are requested right after the plan, when the ring is empty.)
constexpr int kTickets = kPositions;
constexpr unsigned kFrozen = 0x10000u;

// shared-memory map (bytes)
constexpr int kOffRing = 0;
constexpr int kOffAct = kOffRing + kRingSlots * kSlotBytes;                        // 196608
constexpr int kActBytes = (kTopK + 1) * kInter * 2 + 16;                           // 9 x 512 BF16 + gate logit
constexpr int kOffDots = kOffAct + kActBytes;                                      // +9232
constexpr int kOffX = kOffDots + kDecodeMaxRowsPerBlock * kDotsStride * 4;         // +672: layer input, packed BF16
constexpr int kOffNorm = kOffX + kHidden * 2;                                      // +4096: norm weight row
constexpr int kOffMisc = kOffNorm + kHidden * 2;                                   // +4096
constexpr int kMiscBytes = 1024;
constexpr int kOffBars = kOffMisc + kMiscBytes;
constexpr int kBarCount = 2 * kRingSlots + 1;
constexpr int kSmemTotal = kOffBars + kBarCount * 8;
static_assert(kSmemTotal <= 227 * 1024, "decode kernel shared memory exceeds 227 KB");
static_assert(kSmemTotal == kDecodeSmemBytes, "keep decode_kernel.cuh in step");
static_assert(kDecodeMaxRowsPerBlock * kDownRowBytes <= kHalfBytes, "a block's down rows of one expert must fit half a slot");
static_assert((kInter + kDecodeMinBlocks - 1) / kDecodeMinBlocks <= kGroupWarps, "a chunk has at most one row per warp of a group");
static_assert(kGroupWarps * kRowBytes <= kHalfBytes, "a chunk of weight rows must fit half a slot");
static_assert(kStreamWarps + 1 == kDecodeConsumerWarps, "control warp + stream warps meet at the consumer barrier");
static_assert(kRingSlots % kGroups == 0, "every group owns the same number of slots");
static_assert(kDecodeMinBlocks > kRouterBlocks, "block 128 must exist: it carries the shared gate row");

struct Misc {
  int ids[kTopK];                 // selected experts in selection order (rank r)
  float weights[kTopK];           // BF16-rounded routing weights as FP32
  int local_rank[kTopK];          // ranks whose expert lives on this GPU, ascending
  int n_local;
  // ---- layer plan: which expert each ring position carries ----
  int expert_of_pos[kPositions];  // chosen expert dealt to position q, -1: position unused
  int rank_of_pos[kPositions];    // its selection rank
  int pred_of_pos[kPositions];    // expert the blind items of position q were requested with, -1: none
  int active_pos[kPositions];     // used positions, ascending
  int n_active;
  unsigned active_mask;           // bit q: position q carries a chosen expert
  unsigned valid_mask;            // bit q: the blind items of position q hold that expert's rows
  int n_blind;                    // tickets [0, n_blind) were handled blind
  volatile int plan_layer;        // (layer ordinal + 1) the plan above belongs to
  // ---- prediction ----
  int pred[2][kPositions];        // predicted experts of layer ordinal li at [li & 1], -1: not held here
  volatile int pred_layer;        // predictions are published for all layer ordinals < pred_layer
  unsigned blind_state[2];        // [li & 1]: tickets claimed blind so far | kFrozen
  volatile int blind_done[2];     // [li & 1]: tickets the producer has dealt with (placed or skipped)
  uint16_t spec_bits[kStreamWarps][kPositions];   // activations computed blind, published once the plan confirms them
  volatile int abort_flag;        // block-local copy of a raised status
};
static_assert(sizeof(Misc) <= kMiscBytes, "Misc too large");

__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" :: "n"(kDecodeConsumerThreads) : "memory");
}

// (These two take the status pointer, not the parameter block: a reference to the kernel's parameters handed
// to an out-of-line function makes every thread copy the whole block to its stack at kernel entry.)
__device__ __noinline__ void raise_status(int* status, volatile int* abort_flag, int code) {
  atomicCAS(status, 0, code);
  *abort_flag = code;
}

// Records where the first bounded wait gave up: status[1] = site, [2] = block,
// [3] = warp, [4] = item / layer detail.  Sites: 1 producer slot acquire,
// 2 consumer item (router / shared rows), 3 consumer item (routed rows),
// 4 consumer item (down rows), 5 activation exchange, 6 plan hand-over to the producer,
// 7 output exchange, 8 norm row, 9 logits exchange, 10 prediction hand-over,
// 11 expert-parallel peer word, 12 predicted-logits exchange.
__device__ __noinline__ void record_site(int* status, int site, int detail,
                                         const unsigned* diag = nullptr) {
  if (atomicCAS(status + 1, 0, site) == 0) {
    status[2] = blockIdx.x;
    status[3] = threadIdx.x >> 5;
    status[4] = detail;
    if (diag != nullptr) {
      status[5] = static_cast<int>(diag[0]);
      status[6] = static_cast<int>(diag[1]);
      status[7] = static_cast<int>(diag[2]);
      status[8] = static_cast<int>(diag[3]);
    }
  }
}

// Block-uniform verdict on whether any thread of the block has raised a status.
// abort_flag can be set at any moment (e.g. by the producer warp), so consumer
// threads must not branch on their own reading of it around a named barrier.
// One barrier that also reduces: every thread contributes its own sample (a
// thread that raised a status itself sees it), all receive the conjunction.
// (Thread 0 sampling between two barriers: 0.5333 -> 0.5331 ms per token.)
__device__ __forceinline__ bool uniform_alive(volatile int* abort_flag) {
  const int healthy = (*abort_flag == 0) ? 1 : 0;
  int verdict;
  asm volatile(
      "{\n"
      ".reg .pred mine, all;\n"
      "setp.ne.s32 mine, %1, 0;\n"
      "bar.red.and.pred all, 1, %2, mine;\n"
      "selp.s32 %0, 1, 0, all;\n"
      "}\n"
      : "=r"(verdict) : "r"(healthy), "n"(kDecodeConsumerThreads) : "memory");
  return verdict != 0;
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
__device__ __forceinline__ uint32_t ld_strong_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Exchange words are WRITTEN with an atomic exchange whose result nobody reads, not with a store: an atomic is
// performed at L2 as soon as it gets there, while a relaxed store was seen by the pollers of other blocks a
// median 2 us after it was issued (one poll takes 0.27 us) -- three hand-overs per layer made that 8 % of the
// token time (0.682 -> 0.628 ms per token, A/B inside one call; st.volatile: no change; st.release: 1.56 ms).
__device__ __forceinline__ void st_strong_u64(void* p, unsigned long long v) {
  unsigned long long previous;
  asm volatile("atom.relaxed.gpu.global.exch.b64 %0, [%1], %2;" : "=l"(previous) : "l"(p), "l"(v) : "memory");
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
  uint32_t previous;
  asm volatile("atom.relaxed.gpu.global.exch.b32 %0, [%1], %2;" : "=r"(previous) : "l"(p), "r"(v) : "memory");
}

// The 512 rows of a projection are dealt to the blocks as contiguous ranges of 3 or 4 (at 148 blocks):
// range b covers rows [512 b / G, 512 (b + 1) / G).  For the routed experts the range a block takes
// depends on the expert position, so that every block holds 27 or 28 rows in all whatever experts
// the positions carry.
__device__ __forceinline__ int range_lo(int b, int G) { return (b * kInter) / G; }
__device__ __forceinline__ int position_range(int q, int c, int G) {
  int b = c + (q * G) / kPositions;
  if (b >= G) b -= G;
  return b;
}

// Iterative arg-max over 256 keys (8 per lane: key q of lane l belongs to expert 32 q + l), ties to
// the lowest expert id; lane r < 8 ends up with the r-th selection.  Consumes k.
__device__ __forceinline__ void warp_top8(uint32_t (&k)[8], int lane, float& my_score, int& my_id) {
  my_score = 0.0f;
  my_id = 0;
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
}

}  // namespace

// kEp: expert parallelism (world > 1).  kExtras: qualification outputs, tracing stamps and the harness's
// router hooks.  The plain single-GPU instantiation carries neither: its per-layer code runs once per
// layer, so what it does not execute should not be in its text either.
template <bool kEp, bool kExtras>
__global__ void __launch_bounds__(kDecodeThreads, 1)
moe_decode_persistent_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem + kOffRing;
  uint16_t* act_s = reinterpret_cast<uint16_t*>(smem + kOffAct);
  float* dots = reinterpret_cast<float*>(smem + kOffDots);
  uint8_t* x_s = smem + kOffX;
  uint8_t* norm_s = smem + kOffNorm;
  Misc* misc = reinterpret_cast<Misc*>(smem + kOffMisc);
  const uint32_t bars = smem_u32(smem + kOffBars);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kRingSlots + s); };
  const uint32_t norm_bar = bars + 8u * (2 * kRingSlots);

  const int G = gridDim.x;
  const int c = blockIdx.x;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &misc->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRingSlots; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kGroupWarps);
    }
    mbar_init(norm_bar, 1);
    // every ring slot starts out released: complete phase 0 of its empty barrier
    for (int s = 0; s < kRingSlots; ++s)
      for (int m = 0; m < kGroupWarps; ++m) mbar_arrive(empty_bar(s));
    misc->plan_layer = 0;
    misc->pred_layer = 1;          // layer ordinal 0 has no prediction: nothing to wait for
    misc->blind_state[0] = 0u;
    misc->blind_state[1] = 0u;
    misc->blind_done[0] = 0;
    misc->blind_done[1] = 0;
    misc->abort_flag = 0;
    misc->n_local = 0;
    misc->n_active = 0;
    mbar_fence_init();
  }
  __syncthreads();

  const int h0 = (c * kHidden) / G;
  const int h1 = ((c + 1) * kHidden) / G;
  const int nh = h1 - h0;
  const int half_rows = (nh + 1) / 2;
  const bool has_router_rows = c < kRouterBlocks;          // router rows 2c, 2c + 1
  const bool owns_gate_row = (c == kRouterBlocks);         // shared expert's gate row
  const bool has_r1 = has_router_rows || owns_gate_row;
  const int sh_lo = range_lo(c, G);                        // shared-expert input rows [sh_lo, sh_hi)
  const int sh_rows = range_lo(c + 1, G) - sh_lo;
  const bool speculate = p.speculate != 0;
  const unsigned epoch0 = *p.epoch_base;      // exchange tag of layer ordinal li is epoch0 + li + 1
  unsigned long long* const pred_logits = p.logits + kDecodeReplicas * kExperts;

  if (warp == kProducerWarp) {
    // ------------------------------ producer ------------------------------
    // Lanes 0 and 1 walk the same item sequence; lane 0 announces an item's bytes and issues the
    // copy into half A, lane 1 the copy into half B, so two copies are placed at a time.
    if (lane < 2) {
      constexpr unsigned kPair = 0x3u;
      unsigned seq = 0;
      unsigned issued[kRingSlots];
      for (int s = 0; s < kRingSlots; ++s) issued[s] = 0;
      unsigned norm_issued = 0;
      unsigned landed = 0;           // items [0, landed) are known to have arrived
      bool alive = true;

      // One item: `bytes_a` from src_a into half A, `bytes_b` from src_b into half B (either may be 0,
      // not both).  Returns false after a failed wait (both lanes agree).
      auto issue = [&](const void* src_a, uint32_t bytes_a, const void* src_b, uint32_t bytes_b) -> bool {
        const int s = seq % kRingSlots;
        const unsigned use = seq / kRingSlots;
        unsigned diag[4] = {0, 0, 0, 0};
        bool ok = true;
        // Requests queue in the SM's path to L2, and every small load or store of the block -- the polls
        // and stores of the grid-wide hand-overs -- waits behind them: no more than max_in_flight items
        // are outstanding at a time (enough to cover bandwidth x latency, not more).
        if (p.max_in_flight > 0) {
          while (ok && seq - landed >= static_cast<unsigned>(p.max_in_flight)) {
            ok = mbar_wait_bounded(full_bar(landed % kRingSlots), (landed / kRingSlots) & 1u, abort_flag, diag);
            ++landed;
          }
        }
        ok = ok && mbar_wait_bounded(empty_bar(s), use & 1u, abort_flag, diag);
        if (!ok && lane == 0 && *abort_flag == kStatusTimeoutMbarrier) {
          atomicCAS(p.status, 0, kStatusTimeoutMbarrier);
          record_site(p.status, 1, static_cast<int>(seq), diag);
        }
        ok = __all_sync(kPair, ok);
        if (!ok) { alive = false; return false; }
        const uint32_t dst = smem_u32(ring + s * kSlotBytes);
        if (lane == 0) mbar_arrive_expect_tx(full_bar(s), bytes_a + bytes_b);
        __syncwarp(kPair);
        if (lane == 0 && bytes_a != 0u) bulk_g2s(dst, src_a, bytes_a, full_bar(s));
        if (lane == 1 && bytes_b != 0u) bulk_g2s(dst + kHalfBytes, src_b, bytes_b, full_bar(s));
        issued[s] = seq / kRingSlots + 1;
        ++seq;
        return true;
      };
      // bounded wait for a hand-over word in shared memory to reach `want`
      auto wait_word = [&](volatile int* word, int want, int code, int site, int detail) -> bool {
        bool ok = true;
        if (*word < want) {
          const unsigned long long start = global_timer_ns();
          unsigned spins = 0;
          while (*word < want) {
            if ((++spins & 255u) == 0u) {
              if (*abort_flag != 0) { ok = false; break; }
              if (global_timer_ns() - start > kWaitBudgetNs) {
                raise_status(p.status, abort_flag, code);
                record_site(p.status, site, detail);
                ok = false;
                break;
              }
            }
          }
        }
        ok = __all_sync(kPair, ok);
        if (!ok) alive = false;
        return ok;
      };

      // producer-side tracing stamps: 12 router / shared items placed, 13 blind issue over, 14 last
      // gate/up chunk placed, 15 last down item placed
      auto stamp = [&](int li, int k) {
        if (kExtras && p.timeline != nullptr && lane == 0)
          p.timeline[(static_cast<size_t>(c) * kMaxLayers + li) * kDecodeTraceSlots + k] = global_timer_ns();
      };
      for (int li = 0; li < p.n_layers && alive; ++li) {
        const LayerPtrs L = p.layers[p.first_layer + li];
        const bool has_next = speculate && (li + 1 < p.n_layers);
        // the block's chunk of expert `expert` for position q: gate rows into half A, up rows into half B
        auto issue_chunk = [&](int expert, int q) -> bool {
          const int b = position_range(q, c, G);
          const int lo = range_lo(b, G);
          const uint32_t bytes = static_cast<uint32_t>(range_lo(b + 1, G) - lo) * kRowBytes;
          const __nv_bfloat16* gate_rows = L.expert_gate_up +
              (static_cast<size_t>(expert - p.expert_lo) * (2 * kInter) + lo) * kHidden;
          return issue(gate_rows, bytes, gate_rows + static_cast<size_t>(kInter) * kHidden, bytes);
        };
        // ---- norm weight row into its own region (its readers finished before the plan of the
        //      previous layer was published, which this thread has waited for) ----
        if (lane == 0) {
          mbar_arrive_expect_tx(norm_bar, kRowBytes);
          bulk_g2s(smem_u32(norm_s), L.norm_weight, kRowBytes, norm_bar);
        }
        norm_issued = li + 1;
        // ---- R1: router rows (+ the next layer's), or the shared gate row; R2: shared input rows ----
        if (has_r1) {
          const __nv_bfloat16* src_a = has_router_rows ? L.router + static_cast<size_t>(2 * c) * kHidden : L.shared_gate;
          const uint32_t bytes_a = has_router_rows ? 2 * kRowBytes : kRowBytes;
          const bool predict_rows = has_next && has_router_rows;
          const __nv_bfloat16* src_b =
              predict_rows ? p.layers[p.first_layer + li + 1].router + static_cast<size_t>(2 * c) * kHidden : nullptr;
          if (!issue(src_a, bytes_a, src_b, predict_rows ? 2 * kRowBytes : 0u)) break;
        }
        if (sh_rows > 0) {
          if (!issue(L.shared_gate_proj + static_cast<size_t>(sh_lo) * kHidden, sh_rows * kRowBytes,
                     L.shared_up_proj + static_cast<size_t>(sh_lo) * kHidden, sh_rows * kRowBytes)) break;
        }
        stamp(li, 12);
        // ---- B items: gate/up chunks of the predicted experts, until the real routing is known ----
        if (speculate && li > 0) {
          if (!wait_word(&misc->pred_layer, li + 1, kStatusTimeoutIds, 10, li)) break;
          __threadfence_block();
          unsigned* state = &misc->blind_state[li & 1];
          const int* pred = misc->pred[li & 1];
          while (alive) {
            unsigned ticket = 0u;
            if (lane == 0) ticket = atomicAdd(state, 1u);
            ticket = __shfl_sync(kPair, ticket, 0);
            if ((ticket & kFrozen) != 0u || ticket >= static_cast<unsigned>(kTickets)) break;
            const int q = static_cast<int>(ticket);
            if (pred[q] >= 0) issue_chunk(pred[q], q);
            // the ticket is dealt with (its copies are on their way, or there was nothing to copy)
            __syncwarp(kPair);
            if (lane == 0) {
              __threadfence_block();
              misc->blind_done[li & 1] = q + 1;
            }
          }
          if (!alive) break;
        }
        stamp(li, 13);
        // ---- wait for this layer's plan ----
        if (!wait_word(&misc->plan_layer, li + 1, kStatusTimeoutIds, 6, li)) break;
        __threadfence_block();
        const int n_blind = misc->n_blind;
        const unsigned active_mask = misc->active_mask;
        const unsigned valid_mask = misc->valid_mask;
        // ---- P items: chunks not handled blind, then chunks whose blind item holds the wrong expert ----
#pragma unroll 1
        for (int q = n_blind; q < kPositions && alive; ++q) {
          if (((active_mask >> q) & 1u) != 0u) issue_chunk(misc->expert_of_pos[q], q);
        }
#pragma unroll 1
        for (int q = 0; q < n_blind && alive; ++q) {
          if (((active_mask >> q) & 1u) != 0u && ((valid_mask >> q) & 1u) == 0u) issue_chunk(misc->expert_of_pos[q], q);
        }
        if (!alive) break;
        stamp(li, 14);
        // ---- D items: the block's rows of the down projections, two experts per item, shared expert first ----
        const uint32_t down_bytes = static_cast<uint32_t>(nh) * kDownRowBytes;
        const int n_active = misc->n_active;
#pragma unroll 1
        for (int e = 0; e < 1 + n_active && alive; e += 2) {
          const __nv_bfloat16* src[2] = {nullptr, nullptr};
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const int entry = e + k;
            if (entry == 0) {
              src[k] = L.shared_down_proj + static_cast<size_t>(h0) * kInter;
            } else if (entry <= n_active) {
              const int expert = misc->expert_of_pos[misc->active_pos[entry - 1]];
              src[k] = L.expert_down + (static_cast<size_t>(expert - p.expert_lo) * kHidden + h0) * kInter;
            }
          }
          issue(src[0], down_bytes, src[1], src[1] != nullptr ? down_bytes : 0u);
        }
        stamp(li, 15);
      }
      // Drain: every copy these lanes issued must have landed before the block
      // may exit (bounded; a phase that already completed returns at once).
      if (*abort_flag != 0 && lane == 0) {
        for (int s = 0; s < kRingSlots; ++s) {
          if (issued[s] != 0) {
            volatile int ignore = 0;
            mbar_wait_bounded(full_bar(s), (issued[s] - 1u) & 1u, &ignore);
          }
        }
        if (norm_issued != 0) {
          volatile int ignore = 0;
          mbar_wait_bounded(norm_bar, (norm_issued - 1u) & 1u, &ignore);
        }
      }
    }
    __syncwarp();
  } else if (warp == kPredictWarp) {
    // ------------------------------ prediction ----------------------------
    // Top-8 of the next layer's router applied to this layer's input; the ids go to the producer,
    // which requests their rows while this layer's tail and the next layer's head are running.
    if (speculate) {
      for (int li = 0; li + 1 < p.n_layers; ++li) {
        // sleep until this block's own plan for layer li exists: the predicted logits were written
        // right after the real ones, so they are (nearly) complete by then and few polls are needed
        {
          const unsigned long long start = global_timer_ns();
          bool ok = true;
          while (misc->plan_layer < li + 1) {
            __nanosleep(200);
            if (*abort_flag != 0 || global_timer_ns() - start > 2 * kWaitBudgetNs) { ok = false; break; }
          }
          if (!ok) break;
        }
        const unsigned tag = epoch0 + li + 1;
        unsigned long long w[8];
        bool ready = false;
        const unsigned long long start = global_timer_ns();
        unsigned spins = 0;
        while (!ready) {
          bool mine = true;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            w[q] = ld_strong_u64(pred_logits + (c % kDecodeReplicas) * kExperts + 32 * q + lane);
            mine = mine && static_cast<unsigned>(w[q] >> 32) == tag;
          }
          ready = __all_sync(0xffffffffu, mine);
          if (!ready) {
            __nanosleep(100);
            if ((++spins & 15u) == 0u) {
              if (*abort_flag != 0) break;
              if (global_timer_ns() - start > kWaitBudgetNs) {
                raise_status(p.status, abort_flag, kStatusTimeoutPeer);
                record_site(p.status, 12, li);
                break;
              }
            }
          }
        }
        if (!ready) break;
        uint32_t k[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) k[q] = order_key(__uint_as_float(static_cast<uint32_t>(w[q])));
        float score;
        int id;
        warp_top8(k, lane, score, id);
        if (lane < kPositions)
          misc->pred[(li + 1) & 1][lane] = (id >= p.expert_lo && id < p.expert_hi) ? id : -1;
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          misc->pred_layer = li + 2;
        }
      }
    }
    __syncwarp();
  } else if (warp == kControlWarp || (warp & 3) != 0) {
    // ------------------------------ consumers -----------------------------
    const bool streams = warp != kControlWarp;
    const int stream_index = (warp >> 2) * 3 + (warp & 3) - 1;      // 0 .. 11 over warps 1,2,3,5,6,7,...
    const int cw = streams ? 1 + stream_index : 0;                  // consumer warp ordinal 0 .. 12
    const int ctid = cw * 32 + lane;                                // 0 .. 415
    const int group = streams ? stream_index / kGroupWarps : -1;
    const int member = streams ? stream_index % kGroupWarps : -1;
    unsigned seq = 0;                             // mirrors the producer's item counter
    bool alive = true;

    auto owns = [&](unsigned item) -> bool {
      return static_cast<int>((item % kRingSlots) % kGroups) == group;
    };
    // wait for item `item`, return slot pointer (nullptr on abort)
    auto wait_item = [&](unsigned item, int site) -> const uint8_t* {
      const int s = item % kRingSlots;
      const unsigned use = item / kRingSlots;
      unsigned diag[4] = {0, 0, 0, 0};
      if (!mbar_wait_bounded(full_bar(s), use & 1u, abort_flag, diag)) {
        if (*abort_flag == kStatusTimeoutMbarrier) {
          atomicCAS(p.status, 0, kStatusTimeoutMbarrier);
          record_site(p.status, site, static_cast<int>(item), diag);
        }
        return nullptr;
      }
      return ring + s * kSlotBytes;
    };
    auto release_item = [&](unsigned item) {
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(item % kRingSlots));
    };
    // Canonical 2048-dot of the normalised input against one row / two rows at once; the caller merges the
    // lanes' partials with butterfly_sum after it has handed the slot back.  The input is read from shared
    // memory (FP32, two float4 per lane and step) in loops unrolled twice: held in 64 registers per thread and
    // fully unrolled, the same dots took 8 % more time per token (the kernel then sat at its cap of 128
    // registers); four- or eight-fold unrolling is 1 % slower than twofold, no unrolling 2 %.
    auto row_dot = [&](const uint8_t* row, const float4* xq) -> float {
      float a = 0.0f;
      const uint4* r0 = reinterpret_cast<const uint4*>(row) + lane;
#pragma unroll 2
      for (int i = 0; i < 8; ++i) {
        const float4 xlo = xq[i * 32], xhi = xq[256 + i * 32];
        const float x8[8] = {xlo.x, xlo.y, xlo.z, xlo.w, xhi.x, xhi.y, xhi.z, xhi.w};
        a = fma8(x8, r0[i * 32], a);
      }
      return a;
    };
    auto pair_dot = [&](const uint8_t* row_a, const uint8_t* row_b, const float4* xq, float& a, float& b) {
      a = 0.0f; b = 0.0f;
      const uint4* r0 = reinterpret_cast<const uint4*>(row_a) + lane;
      const uint4* r1 = reinterpret_cast<const uint4*>(row_b) + lane;
#pragma unroll 2
      for (int i = 0; i < 8; ++i) {
        const uint4 w0 = r0[i * 32];
        const uint4 w1 = r1[i * 32];
        const float4 xlo = xq[i * 32], xhi = xq[256 + i * 32];
        const float x8[8] = {xlo.x, xlo.y, xlo.z, xlo.w, xhi.x, xhi.y, xhi.z, xhi.w};
        a = fma8(x8, w0, a);
        b = fma8(x8, w1, b);
      }
    };
    auto hooked_logit = [&](float v, int expert) -> float {
      if (kExtras && p.router_bias != nullptr) v = __fadd_rn(v, p.router_bias[expert]);
      if (kExtras && p.quant_eighths) v = __fmul_rn(rintf(__fmul_rn(v, 8.0f)), 0.125f);
      return v;
    };

    // tracing stamps (thread 0 of the block unless stated): 0 layer start, 1 norm done, 2 this block's
    // logits written (by the warp that computed them), 3 all logits arrived, 4 plan published and blind
    // chunks consumed, 5 routed gate/up done, 6 activations of all blocks polled and packed, 7 block agrees to go on, 8 first down
    // item of the first streaming warp has landed, 9 down dots done, 10 output stored, 11 that warp's
    // down items done
    auto stamp_now = [&](int li, int k) {
      if (kExtras && p.timeline != nullptr)
        p.timeline[(static_cast<size_t>(c) * kMaxLayers + li) * kDecodeTraceSlots + k] = global_timer_ns();
    };
    auto stamp = [&](int li, int k) {
      if (ctid == 0) stamp_now(li, k);
    };
    if (p.n_layers > 1) {
      // The output words between the layers of a launch are only written by launches of several layers, while
      // every launch advances the epoch: a word left by such a launch 65 535 epochs ago carries the tag this
      // launch expects.  Every block therefore clears the words it writes (its output rows, every copy, both
      // buffers) before anything else; a reader gets to them only after this block's logits and activations
      // of the first layer, which come later in program order.
      if (ctid < nh) {
#pragma unroll
        for (int rep = 0; rep < kDecodeReplicas; ++rep) {
          st_strong_u32(p.xbuf0 + rep * kHidden + h0 + ctid, 0u);
          st_strong_u32(p.xbuf1 + rep * kHidden + h0 + ctid, 0u);
        }
      }
      __threadfence();
    }
    if (kEp) {
      // Expert parallelism leaves the activation words of positions this GPU does not use unwritten, possibly
      // for many calls, and a 16-bit tag comes round again: every call starts by clearing the words this block
      // writes (its up to four columns of every position, in every copy), before any of its own stores to them.
      if (ctid < kPositions * kDecodeReplicas * 4) {
        const int q = ctid / (kDecodeReplicas * 4);
        const int rep = (ctid / 4) % kDecodeReplicas;
        const int m = ctid & 3;
        const int b = position_range(q, c, G);
        const int lo = range_lo(b, G);
        if (m < range_lo(b + 1, G) - lo) st_strong_u32(p.act + rep * kDecodeActStride + q * kInter + lo + m, 0u);
      }
      __threadfence();
      consumer_sync();
    }
#pragma unroll 1
    for (int li = 0; li < p.n_layers; ++li) {
      const bool first = (li == 0);
      const bool last = (li == p.n_layers - 1);
      const bool has_next = speculate && !last;

      stamp(li, 0);
      const uint32_t* xw_src = (li & 1) ? p.xbuf1 : p.xbuf0;     // tagged words written by layer li - 1
      uint32_t* xw_dst = (li & 1) ? p.xbuf0 : p.xbuf1;
      // 16-bit tags that are never zero (a cleared word matches no layer): ((epoch) mod 65535) + 1
      const unsigned tag_in = ((epoch0 + static_cast<unsigned>(li)) % 0xffffu) + 1u;           // tag of layer li - 1
      const unsigned tag_out = ((epoch0 + static_cast<unsigned>(li) + 1u) % 0xffffu) + 1u;
      const uint32_t act_tag = tag_out << 16;                     // activation words of this layer
      // ---- layer input into shared memory (packed BF16) ----
      if (first) {
        if (ctid < kHidden / 8) {
          reinterpret_cast<uint4*>(x_s)[ctid] = ld_cg_u4(reinterpret_cast<const uint4*>(p.x_in) + ctid);
        }
      } else if (cw < 8) {
        // poll this warp's 256 tagged words until every tag is the previous layer's
        const uint4* src = reinterpret_cast<const uint4*>(xw_src + (c % kDecodeReplicas) * kHidden) + cw * 64 + lane;
        uint4 w[2];
        bool ready = false;
        const unsigned long long start = global_timer_ns();
        unsigned spins = 0;
        while (!ready) {
          bool mine = true;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            w[i] = ld_strong_u4(src + i * 32);
            mine = mine && (w[i].x >> 16) == tag_in && (w[i].y >> 16) == tag_in &&
                   (w[i].z >> 16) == tag_in && (w[i].w >> 16) == tag_in;
          }
          ready = __all_sync(0xffffffffu, mine);
          if (!ready && (++spins & 63u) == 0u) {
            if (*abort_flag != 0) break;
            if (global_timer_ns() - start > kWaitBudgetNs) {
              raise_status(p.status, abort_flag, kStatusTimeoutPeer);
              record_site(p.status, 7, li);
              break;
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          uint2 packed;
          packed.x = (w[i].x & 0xffffu) | (w[i].y << 16);
          packed.y = (w[i].z & 0xffffu) | (w[i].w << 16);
          reinterpret_cast<uint2*>(x_s)[cw * 64 + i * 32 + lane] = packed;
        }
      }
      if (!uniform_alive(abort_flag)) break;
      // ---- norm, once per block.  Sum of squares in the order of the reference kernel
      //      (native/src/native_pointwise.hip.cpp:109-142): partial t of 256 adds elements t, t + 256, ...
      //      in that order, the partials fold by halving.  Consumer warp j holds partial 8 l + j on lane l: the
      //      butterfly does the halvings of width 128 .. 8, the last three widths are the tree below.
      //      Then every thread normalises one 8-element chunk into h2_s as FP32 (the activation region is idle now):
      //      chunk t's elements 0..3 at float4 t, elements 4..7 at float4 256 + t, so that a warp's loads of
      //      either half are contiguous
      uint8_t* h2_s = reinterpret_cast<uint8_t*>(act_s);
      if (cw < 8) {
        float acc = 0.0f;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float v = bf16_bits_to_float(reinterpret_cast<const uint16_t*>(x_s)[256 * g + 8 * lane + cw]);
          acc = __fmaf_rn(v, v, acc);
        }
        acc = butterfly_sum(acc);
        if (lane == 0) dots[cw] = acc;
      }
      consumer_sync();
      {
        const float total = __fadd_rn(__fadd_rn(__fadd_rn(dots[0], dots[4]), __fadd_rn(dots[2], dots[6])),
                                      __fadd_rn(__fadd_rn(dots[1], dots[5]), __fadd_rn(dots[3], dots[7])));
        const float inv = det_rsqrtf(__fadd_rn(__fdiv_rn(total, static_cast<float>(kHidden)), p.eps));
        if (!mbar_wait_bounded(norm_bar, li & 1u, abort_flag)) {
          if (*abort_flag == kStatusTimeoutMbarrier) {
            atomicCAS(p.status, 0, kStatusTimeoutMbarrier);
            record_site(p.status, 8, li);
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
          float f[8];
          unpack8(out, f);
          reinterpret_cast<float4*>(h2_s)[ctid] = make_float4(f[0], f[1], f[2], f[3]);
          reinterpret_cast<float4*>(h2_s)[256 + ctid] = make_float4(f[4], f[5], f[6], f[7]);
          if (kExtras && p.dbg_h2 != nullptr && c == 0) reinterpret_cast<uint4*>(p.dbg_h2)[ctid] = out;
        }
      }
      consumer_sync();
      // element k = 256 g + 8 lane + j of the normalised input is component j & 3 of xr[(j >> 2) * 256 + 32 g]
      const float4* xr = reinterpret_cast<const float4*>(h2_s) + lane;

      stamp(li, 1);
      // ---- R1: warp m of the group takes row m of {router 2c, router 2c+1, next router 2c, next router 2c+1};
      //      in block 128 warp 0 takes the shared gate row ----
      if (has_r1) {
        const unsigned item = seq++;
        if (streams && owns(item) && alive) {
          const uint8_t* slot = wait_item(item, 2);
          if (!__all_sync(0xffffffffu, slot != nullptr)) alive = false;
          if (alive) {
            const bool predicted = member >= 2;
            const bool has_row = has_router_rows ? (!predicted || has_next) : (member == 0);
            float v = 0.0f;
            if (has_row) v = row_dot(slot + (predicted ? kHalfBytes : 0) + (member & 1) * kRowBytes, xr);
            release_item(item);
            if (has_row) v = butterfly_sum(v);
            if (has_row && lane == 0) {
              if (has_router_rows) {
                const int expert = 2 * c + (member & 1);
                unsigned long long* dst = predicted ? pred_logits : p.logits;
                const unsigned long long word =
                    (static_cast<unsigned long long>(epoch0 + li + 1) << 32) | __float_as_uint(hooked_logit(v, expert));
#pragma unroll
                for (int rep = 0; rep < kDecodeReplicas; ++rep) st_strong_u64(dst + rep * kExperts + expert, word);
                if (!predicted) stamp_now(li, 2);
              } else {
                const uint32_t word = act_tag | float_to_bf16_bits(v);       // the gate logit is used BF16-rounded
#pragma unroll
                for (int rep = 0; rep < kDecodeReplicas; ++rep)
                  st_strong_u32(p.act + rep * kDecodeActStride + 9 * kInter, word);
              }
            }
          }
        }
      }
      // ---- R2: warp m takes shared-expert input pair sh_lo + m ----
      if (sh_rows > 0) {
        const unsigned item = seq++;
        if (streams && owns(item) && alive) {
          const uint8_t* slot = wait_item(item, 2);
          if (!__all_sync(0xffffffffu, slot != nullptr)) alive = false;
          if (alive) {
            float a = 0.0f, b = 0.0f;
            if (member < sh_rows) pair_dot(slot + member * kRowBytes, slot + kHalfBytes + member * kRowBytes, xr, a, b);
            release_item(item);
            if (member < sh_rows) { a = butterfly_sum(a); b = butterfly_sum(b); }
            if (member < sh_rows && lane == 0) {
              const float g = round_bf16(a);
              const float u = round_bf16(b);
              const uint16_t bits = float_to_bf16_bits(__fmul_rn(det_silu(g), u));
#pragma unroll
              for (int rep = 0; rep < kDecodeReplicas; ++rep)
                st_strong_u32(p.act + rep * kDecodeActStride + kTopK * kInter + sh_lo + member, act_tag | bits);
            }
          }
        }
      }

      // A gate/up chunk for position q: warp m of the owning group takes pair m.  use == false: the
      // slot holds rows of an expert that was not chosen; wait for them to land (the copy must not
      // be in flight when the slot is reused) and hand the slot back unread.  Activations are filed
      // under the POSITION; the down products look the rank up in the plan.
      auto publish_act = [&](int index, uint16_t bits) {
#pragma unroll
        for (int rep = 0; rep < kDecodeReplicas; ++rep) st_strong_u32(p.act + rep * kDecodeActStride + index, act_tag | bits);
      };
      unsigned spec_have = 0u;            // positions whose blind result this warp holds in spec_bits
      auto consume_chunk = [&](int q, bool use, bool blind = false) {
        const unsigned item = seq++;
        if (!streams || !owns(item) || !alive) return;
        const uint8_t* slot = wait_item(item, 3);
        if (!__all_sync(0xffffffffu, slot != nullptr)) { alive = false; return; }
        const int b = position_range(q, c, G);
        const int lo = range_lo(b, G);
        const int rows = range_lo(b + 1, G) - lo;
        const bool mine = use && member < rows;
        float a = 0.0f, bb = 0.0f;
        if (mine) pair_dot(slot + member * kRowBytes, slot + kHalfBytes + member * kRowBytes, xr, a, bb);
        release_item(item);
        if (mine) { a = butterfly_sum(a); bb = butterfly_sum(bb); }
        if (mine && lane == 0) {
          const uint16_t bits = float_to_bf16_bits(__fmul_rn(det_silu(a), bb));
          // a word with this layer's tag is final for its readers: a blind result waits for the plan
          if (blind) misc->spec_bits[stream_index][q] = bits;
          else publish_act(q * kInter + lo + member, bits);
        }
        if (blind && mine) spec_have |= 1u << q;
      };
      // ---- blind gate/up chunks, consumed while warp 0 waits for the logits: the predicted expert's
      //      activations are right whenever the prediction is, and overwritten otherwise.  Every warp
      //      takes the chunks in ticket order until it meets the first ticket that was not claimed
      //      before the routing was known (n_blind, published with the plan) ----
      int blind_seen = 0;                 // gate/up tickets this warp has walked past
      if (speculate && li > 0 && streams) {
        const unsigned long long start = global_timer_ns();
        unsigned spins = 0;
#pragma unroll 1
        while (blind_seen < kPositions && alive) {
          if (misc->blind_done[li & 1] > blind_seen) {
            __threadfence_block();
            if (misc->pred[li & 1][blind_seen] >= 0) consume_chunk(blind_seen, true, true);
            ++blind_seen;
            continue;
          }
          if (misc->plan_layer == li + 1) {
            __threadfence_block();
            if (blind_seen >= misc->n_blind) break;       // never claimed: dealt with after the plan
          }
          if ((++spins & 255u) == 0u) {
            if (*abort_flag != 0) { alive = false; break; }
            if (global_timer_ns() - start > kWaitBudgetNs) {
              raise_status(p.status, abort_flag, kStatusTimeoutIds);
              record_site(p.status, 13, li * 16 + blind_seen);
              alive = false;
              break;
            }
          }
        }
      }

      // ---- logits exchange + top-8 (ties to the lowest expert id) + softmax + layer plan, warp 0 ----
      if (warp == kControlWarp) {
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
              raise_status(p.status, abort_flag, kStatusTimeoutPeer);
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
                if (bad == first_bad) {
                  const unsigned long long word = w[(first_bad >> 5) & 7];
                  unsigned diag[4] = {tag, static_cast<unsigned>(first_bad),
                                      static_cast<unsigned>(n_bad) | (alive ? 0x10000u : 0u), static_cast<unsigned>(word >> 32)};
                  record_site(p.status, 9, li, diag);
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
          if (kExtras && p.dbg_logits != nullptr && c == 0) p.dbg_logits[32 * q + lane] = value;
        }
        float my_score;      // lane r keeps the r-th selected value
        int my_id;
        warp_top8(k, lane, my_score, my_id);
        // The routing is known: stop the blind issue.  The value the counter held says exactly how many
        // positions the producer has claimed blind (it may still be placing the last of them).
        unsigned claimed = 0u;
        if (lane == 0) {
          claimed = atomicOr(&misc->blind_state[li & 1], kFrozen) & (kFrozen - 1u);
          misc->blind_state[(li + 1) & 1] = 0u;      // nobody uses the other words before this layer's plan
          misc->blind_done[(li + 1) & 1] = 0;
        }
        claimed = __shfl_sync(0xffffffffu, claimed, 0);
        const int n_blind = min(static_cast<int>(claimed), kTickets);
        // softmax over the eight: exp(s_r - s_0) / sum, summed in selection order
        const float top = __shfl_sync(0xffffffffu, my_score, 0);
        const float ex = det_expf(__fsub_rn(my_score, top));
        float denom = 0.0f;
#pragma unroll
        for (int r = 0; r < kTopK; ++r) denom = __fadd_rn(denom, __shfl_sync(0xffffffffu, ex, r));
        const uint16_t wb = float_to_bf16_bits(__fdiv_rn(ex, denom));
        const bool local_expert = lane < kTopK && my_id >= p.expert_lo && my_id < p.expert_hi;
        const unsigned local_mask = __ballot_sync(0xffffffffu, local_expert);
        // ---- deal the chosen experts held here to the ring positions: an expert the prediction placed
        //      at a position stays there; the others take the remaining positions in ascending order.
        //      Activations are filed by position, so this assignment must be the same in every block:
        //      it uses the whole prediction (identical everywhere), not only the part this block had
        //      claimed blind before the routing was known ----
        int pred_all = -1;
        if (speculate && li > 0) {
          // the prediction for this layer was published during the previous one; make sure of it
          const unsigned long long wait_start = global_timer_ns();
          while (misc->pred_layer < li + 1) {
            if (*abort_flag != 0 || global_timer_ns() - wait_start > kWaitBudgetNs) {
              if (*abort_flag == 0 && lane == 0) {
                raise_status(p.status, abort_flag, kStatusTimeoutIds);
                record_site(p.status, 10, li);
              }
              break;
            }
          }
          __threadfence_block();
          if (lane < kPositions) pred_all = misc->pred[li & 1][lane];
        }
        const int pred_q = lane < n_blind ? pred_all : -1;     // what this block's blind chunks were requested with
        int rank_q = -1;
#pragma unroll
        for (int r = 0; r < kTopK; ++r) {
          const int id_r = __shfl_sync(0xffffffffu, my_id, r);
          if (((local_mask >> r) & 1u) != 0u && pred_all >= 0 && pred_all == id_r) rank_q = r;
        }
        const bool matched = lane < kPositions && rank_q >= 0;
        const unsigned matched_mask = __ballot_sync(0xffffffffu, matched);
        const unsigned matched_ranks = __reduce_or_sync(0xffffffffu, matched ? (1u << rank_q) : 0u);
        // a matched position holds valid rows only if this block had claimed it blind
        const unsigned valid_mask = __ballot_sync(0xffffffffu, matched && lane < n_blind);
        const unsigned free_pos = ((1u << kPositions) - 1u) & ~matched_mask;
        if (lane < kPositions && !matched) {
          unsigned left = local_mask & ~matched_ranks;
          const int skip = __popc(free_pos & ((1u << lane) - 1u));
          for (int t = 0; t < skip && left != 0u; ++t) left &= left - 1u;
          rank_q = left != 0u ? __ffs(left) - 1 : -1;
        }
        const int expert_q = __shfl_sync(0xffffffffu, my_id, rank_q >= 0 ? rank_q : 0);
        const unsigned active_mask = __ballot_sync(0xffffffffu, lane < kPositions && rank_q >= 0);
        if (lane < kTopK) {
          misc->ids[lane] = my_id;
          misc->weights[lane] = bf16_bits_to_float(wb);
          if (local_expert) misc->local_rank[__popc(local_mask & ((1u << lane) - 1u))] = lane;
          misc->expert_of_pos[lane] = rank_q >= 0 ? expert_q : -1;
          misc->rank_of_pos[lane] = rank_q;
          misc->pred_of_pos[lane] = pred_q;
          if (rank_q >= 0) misc->active_pos[__popc(active_mask & ((1u << lane) - 1u))] = lane;
          if (c == 0) {
            if (kExtras && p.dbg_ids != nullptr) p.dbg_ids[lane] = my_id;
            if (kExtras && p.dbg_scores != nullptr) p.dbg_scores[lane] = my_score;
            if (kExtras && p.dbg_weights != nullptr) reinterpret_cast<uint16_t*>(p.dbg_weights)[lane] = wb;
          }
        }
        __syncwarp();
        if (lane == 0) {
          misc->n_local = __popc(local_mask);
          misc->n_active = __popc(active_mask);
          misc->active_mask = active_mask;
          misc->valid_mask = valid_mask;
          misc->n_blind = n_blind;
          __threadfence_block();
          misc->plan_layer = li + 1;
        }
      }
      if (!uniform_alive(abort_flag)) break;
      stamp(li, 4);

      // ---- routed gate/up chunks that were not (or wrongly) covered blind ----
      const int n_local = misc->n_local;
      const int n_blind = misc->n_blind;
      const int n_blind_chunks = n_blind;
      const int n_active = misc->n_active;
      const unsigned active_mask = misc->active_mask;
      const unsigned valid_mask = misc->valid_mask;
      if (streams && lane == 0) {
        // blind results the plan has confirmed
        unsigned confirmed = spec_have & valid_mask;
        while (confirmed != 0u) {
          const int q = __ffs(confirmed) - 1;
          confirmed &= confirmed - 1u;
          publish_act(q * kInter + range_lo(position_range(q, c, G), G) + member, misc->spec_bits[stream_index][q]);
        }
      }
      if (warp == kControlWarp) {
        // warp 0 took no part in the blind walk: count the items it skipped
        for (int q = 0; q < n_blind_chunks; ++q) {
          if (misc->pred_of_pos[q] >= 0) ++seq;
        }
      } else {
        // tickets claimed blind that this warp had not reached when it left the walk above
#pragma unroll 1
        for (; blind_seen < n_blind_chunks; ++blind_seen) {
          if (misc->pred_of_pos[blind_seen] >= 0) consume_chunk(blind_seen, ((valid_mask >> blind_seen) & 1u) != 0u);
        }
      }
#pragma unroll 1
      for (int q = n_blind_chunks; q < kPositions; ++q) {
        if (((active_mask >> q) & 1u) != 0u) consume_chunk(q, true);
      }
#pragma unroll 1
      for (int q = 0; q < n_blind_chunks; ++q) {
        if (((active_mask >> q) & 1u) != 0u && ((valid_mask >> q) & 1u) == 0u) consume_chunk(q, true);
      }
      consumer_sync();
      stamp(li, 5);
      // ---- activation exchange: every block polls the tagged words of the used positions and of the shared
      //      expert (four words = four activations per load, up to three loads per thread) until all carry this
      //      layer's tag, and packs them into shared memory.  No barrier: the words are the synchronisation.
      //      A word of layer li + 1 is written only after its writer has seen every block's output of layer li,
      //      so nobody still waits for layer li's words then ----
      {
        constexpr int kGroups4 = (kTopK + 1) * kInter / 4;                       // 1152 groups of four words
        constexpr int kPerThread = (kGroups4 + kDecodeConsumerThreads - 1) / kDecodeConsumerThreads;
        const uint32_t* words = p.act + (c % kDecodeReplicas) * kDecodeActStride;
        const unsigned tag16 = act_tag >> 16;
        bool need[kPerThread];
#pragma unroll
        for (int i = 0; i < kPerThread; ++i) {
          const int v = ctid + i * kDecodeConsumerThreads;
          const int row = v / (kInter / 4);
          need[i] = v < kGroups4 && (row == kTopK || ((active_mask >> row) & 1u) != 0u);
        }
        uint4 w[kPerThread];
        bool pending[kPerThread];          // a group of words is asked for again only until it has arrived
#pragma unroll
        for (int i = 0; i < kPerThread; ++i) pending[i] = need[i];
        uint32_t gate_word = 0u;
        bool gate_pending = ctid == 0;
        bool ready = false;
        const unsigned long long start = global_timer_ns();
        unsigned spins = 0;
        while (!ready) {
          bool mine = true;
#pragma unroll
          for (int i = 0; i < kPerThread; ++i) {
            if (pending[i]) w[i] = ld_strong_u4(reinterpret_cast<const uint4*>(words) + ctid + i * kDecodeConsumerThreads);
          }
          if (gate_pending) gate_word = ld_strong_u32(words + 9 * kInter);
#pragma unroll
          for (int i = 0; i < kPerThread; ++i) {
            if (pending[i]) {
              pending[i] = !((w[i].x >> 16) == tag16 && (w[i].y >> 16) == tag16 && (w[i].z >> 16) == tag16 &&
                             (w[i].w >> 16) == tag16);
              mine = mine && !pending[i];
            }
          }
          if (gate_pending) {
            gate_pending = (gate_word >> 16) != tag16;
            mine = mine && !gate_pending;
          }
          ready = __all_sync(0xffffffffu, mine);
          if (!ready && (++spins & 63u) == 0u) {
            if (*abort_flag != 0) break;
            if (global_timer_ns() - start > kWaitBudgetNs) {
              raise_status(p.status, abort_flag, kStatusTimeoutPeer);
              record_site(p.status, 5, li);
              break;
            }
          }
        }
#pragma unroll
        for (int i = 0; i < kPerThread; ++i) {
          if (need[i]) {
            uint2 packed;
            packed.x = (w[i].x & 0xffffu) | (w[i].y << 16);
            packed.y = (w[i].z & 0xffffu) | (w[i].w << 16);
            reinterpret_cast<uint2*>(act_s)[ctid + i * kDecodeConsumerThreads] = packed;
          }
        }
        if (ctid == 0) *reinterpret_cast<float*>(act_s + 9 * kInter) = bf16_bits_to_float(static_cast<uint16_t>(gate_word & 0xffffu));
      }
      stamp(li, 6);
      if (!uniform_alive(abort_flag)) break;
      stamp(li, 7);
      {
        // A down item holds the block's rows of up to two experts; warps 0, 1 of the group take the halves
        // of the first expert's rows, warps 2, 3 those of the second: the activation row is unpacked
        // once and up to seven dots against it share one eight-way reduction.  entry 0 is the shared
        // expert, entry e >= 1 position e - 1; use_x == false: that half is absent or holds rows of an
        // expert that was not chosen.
        bool down_stamped = false;
        auto consume_down = [&](int entry_a, bool use_a, int entry_b, bool use_b) {
          const unsigned item = seq++;
          if (!streams || !owns(item) || !alive) return;
          const uint8_t* slot = wait_item(item, 4);
          if (!__all_sync(0xffffffffu, slot != nullptr)) { alive = false; return; }
          if (cw == 1 && lane == 0 && !down_stamped) { stamp_now(li, 8); down_stamped = true; }
          const int entry = (member >> 1) ? entry_b : entry_a;
          const bool mine = (member >> 1) ? use_b : use_a;
          const int act_row = entry == 0 ? kTopK : entry - 1;                       // activations are filed by position
          const int column = (entry == 0 || !mine) ? kTopK : misc->rank_of_pos[entry - 1];
          const int row_base = (member & 1) * half_rows;
          const int rows = mine ? ((member & 1) ? nh - half_rows : half_rows) : 0;
          float part[8];
          if (mine) {
            float af[16];
            const uint4* arow = reinterpret_cast<const uint4*>(act_s + act_row * kInter) + lane;
            unpack8(arow[0], af);
            unpack8(arow[32], af + 8);
            const uint8_t* rows_ptr = slot + (member >> 1) * kHalfBytes + row_base * kDownRowBytes;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              float acc = 0.0f;
              if (u < rows) {
                const uint4* wrow = reinterpret_cast<const uint4*>(rows_ptr + u * kDownRowBytes) + lane;
                acc = fma8(af, wrow[0], acc);
                acc = fma8(af + 8, wrow[32], acc);
              }
              part[u] = acc;
            }
          }
          release_item(item);
          if (mine) {
            const float total = warp_reduce8(part, lane);
            const int u = reduce8_slot(lane);
            if ((lane & 3) == 0 && u < rows) dots[(row_base + u) * kDotsStride + column] = total;
          }
        };
        // entries: 0 the shared expert, e >= 1 the e-th used position
#pragma unroll 1
        for (int e = 0; e < 1 + n_active; e += 2) {
          const int entry_a = e == 0 ? 0 : misc->active_pos[e - 1] + 1;
          const bool has_b = e + 1 <= n_active;
          const int entry_b = has_b ? misc->active_pos[e] + 1 : 0;
          consume_down(entry_a, true, entry_b, has_b);
        }
        if (cw == 1 && lane == 0) stamp_now(li, 11);
      }
      if (!uniform_alive(abort_flag)) break;
      stamp(li, 9);
      // ---- expert parallelism: the down products of the rank slots held here go to every peer
      //      (plain stores over NVLink into its exchange buffer), those held elsewhere are polled
      //      from this GPU's own buffer; words carry the layer tag, buffers alternate per layer.
      //      Block c of every GPU owns the same output rows, so a peer can be at most one layer ahead.
      if (kEp && alive) {
        const unsigned long long tag64 = static_cast<unsigned long long>(epoch0 + li + 1) << 32;
        const size_t parity_base = static_cast<size_t>(li & 1) * kTopK * kHidden;
        const int sends = n_local * nh * (p.world - 1);
        for (int s = ctid; s < sends; s += kDecodeConsumerThreads) {
          const int peer_slot = s / (n_local * nh);
          const int rest = s - peer_slot * (n_local * nh);
          const int q = rest / nh;
          const int hh = rest - q * nh;
          const int peer = peer_slot + (peer_slot >= p.rank ? 1 : 0);
          const int r = misc->local_rank[q];
          st_sys_u64(p.ep_dots[peer] + parity_base + static_cast<size_t>(r) * kHidden + h0 + hh,
                     tag64 | __float_as_uint(dots[hh * kDotsStride + r]));
        }
      }
      if (ctid < nh) {
        const int h = h0 + ctid;
        float acc = 0.0f;
        if (!kEp) {
#pragma unroll
          for (int r = 0; r < kTopK; ++r) {
            const float d = dots[ctid * kDotsStride + r];
            acc = __fmaf_rn(misc->weights[r], d, acc);
            if (kExtras && p.dbg_slot_dots != nullptr) p.dbg_slot_dots[r * kHidden + h] = d;
          }
        } else {
          const unsigned tag = epoch0 + li + 1;
          const unsigned long long* mine = p.ep_dots[p.rank] + static_cast<size_t>(li & 1) * kTopK * kHidden + h;
          int q = 0;
          const unsigned long long start = global_timer_ns();
          for (int r = 0; r < kTopK; ++r) {
            float d;
            if (q < n_local && misc->local_rank[q] == r) {
              d = dots[ctid * kDotsStride + r];
              ++q;
            } else {
              unsigned long long word = ld_sys_u64(mine + static_cast<size_t>(r) * kHidden);
              unsigned spins = 0;
              while (static_cast<unsigned>(word >> 32) != tag) {
                if ((++spins & 63u) == 0u) {
                  if (*abort_flag != 0) break;
                  if (global_timer_ns() - start > kWaitBudgetNs) {
                    raise_status(p.status, abort_flag, kStatusTimeoutPeer);
                    record_site(p.status, 11, li * 16 + r);
                    break;
                  }
                }
                word = ld_sys_u64(mine + static_cast<size_t>(r) * kHidden);
              }
              d = __uint_as_float(static_cast<uint32_t>(word));
            }
            acc = __fmaf_rn(misc->weights[r], d, acc);
            if (kExtras && p.dbg_slot_dots != nullptr) p.dbg_slot_dots[r * kHidden + h] = d;
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
        if (kExtras && p.dbg_routed != nullptr) p.dbg_routed[h] = __float2bfloat16_rn(routed);
        if (kExtras && p.dbg_shared_scaled != nullptr) p.dbg_shared_scaled[h] = __float2bfloat16_rn(shared_scaled);
      }
      stamp(li, 10);
    }
    if (c == 0 && ctid == 0 && *abort_flag == 0) {
      // the counter lives in [0, 65535 * 65536): the 16-bit tags, (epoch mod 65535) + 1, then stay consecutive
      // when it comes round (a plain 32-bit wrap would repeat one tag in two successive layers)
      *p.epoch_base = (epoch0 + static_cast<unsigned>(p.n_layers)) % kDecodeEpochPeriod;
    }
  }
  __syncthreads();
}

namespace {
template <bool kEp, bool kExtras>
cudaError_t launch_variant(const DecodeParams& params, int grid_blocks, cudaStream_t stream) {
  const cudaError_t e = opt_in_dynamic_smem<moe_decode_persistent_kernel<kEp, kExtras>>(kDecodeSmemBytes);
  if (e != cudaSuccess) return e;
  DecodeParams local = params;
  void* args[] = {&local};
  return cudaLaunchCooperativeKernel(
      reinterpret_cast<const void*>(moe_decode_persistent_kernel<kEp, kExtras>), dim3(grid_blocks),
      dim3(kDecodeThreads), args, kDecodeSmemBytes, stream);
}
}  // namespace

cudaError_t launch_moe_decode(const DecodeParams& params, int grid_blocks,
                              cudaStream_t stream) {
  const bool extras = params.timeline != nullptr || params.router_bias != nullptr || params.quant_eighths != 0 ||
                      params.dbg_h2 != nullptr || params.dbg_logits != nullptr || params.dbg_ids != nullptr ||
                      params.dbg_scores != nullptr || params.dbg_weights != nullptr ||
                      params.dbg_shared_scaled != nullptr || params.dbg_routed != nullptr ||
                      params.dbg_slot_dots != nullptr;
  if (params.world > 1) {
    return extras ? launch_variant<true, true>(params, grid_blocks, stream)
                  : launch_variant<true, false>(params, grid_blocks, stream);
  }
  return extras ? launch_variant<false, true>(params, grid_blocks, stream)
                : launch_variant<false, false>(params, grid_blocks, stream);
}

}  // namespace aima
