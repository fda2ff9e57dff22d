// Parameters and launcher of the persistent batch-1 decode kernel.
#pragma once

#include "common.cuh"

namespace aima {

// 16 warps, 4 per SM sub-partition: warp 0 control (exchanges, top-8, layer plan), warp 4 issues the
// bulk copies, warp 8 predicts the next layer's experts, warp 12 is spare, the other twelve stream
// the weight ring.  Warp 0 and the twelve streaming warps form the "consumer" group of 13 warps that
// meets at named barrier 1.
constexpr int kDecodeConsumerWarps = 13;
constexpr int kDecodeConsumerThreads = kDecodeConsumerWarps * 32;
constexpr int kDecodeThreads = 16 * 32;
// Each block owns hidden/grid output elements; their down-projection rows (1 KB each) pass
// through the ring in two items of at most 7 rows per expert: at most 14 rows per block,
// i.e. the grid must have at least ceil(2048 / 14) = 147 blocks.
constexpr int kDecodeMaxRowsPerBlock = 14;
constexpr int kDecodeMinBlocks = (kHidden + kDecodeMaxRowsPerBlock - 1) / kDecodeMaxRowsPerBlock;
constexpr int kDecodeMaxBlocks = kExperts;  // router rows are dealt c, c + grid
constexpr int kDecodeSmemBytes = 215832;
constexpr int kDecodeTraceStamps = 12;       // consumer-side stamps per layer (the public timeline)
constexpr int kDecodeTraceSlots = 16;        // per (block, layer): those 12 + 4 producer-side stamps
constexpr size_t kEpExchangeBytes = 2ull * kTopK * kHidden * 8;   // per-GPU expert-parallel exchange buffer
// Everything all 148 blocks read back from global memory (router logits, the
// activation vector, the layer output) is written kDecodeReplicas times, and
// block c reads copy c % kDecodeReplicas: 148 readers of the same few L2 lines
// otherwise queue at the L2 slices that own them.  Every copy costs its writer
// one atomic, so few copies win: 0.6175 / 0.610 / 0.6175 / 0.628 / 0.650 ms per
// token with 1 / 2 / 4 / 8 / 16 copies (with plain stores, which the pollers saw
// late whatever the count, 8 had been the flat optimum).
constexpr int kDecodeReplicas = 2;
constexpr unsigned kDecodeEpochPeriod = 65535u * 65536u;   // the device-resident epoch counter counts modulo this
// Ring items outstanding per block (0: no limit): before it asks for a slot the producer waits until the item
// issued this many items ago has landed.  0.6105 ms per token without, 0.704 / 0.601 / 0.601 / 0.600 / 0.602 with a
// limit of 1 / 2 / 3 / 4 / 6 (A/B inside one call).
constexpr int kDecodeDefaultInFlight = 4;
constexpr int kDecodeLogitWords = 2 * kDecodeReplicas * kExperts;   // real + predicted, 64-bit words
constexpr int kDecodeActStride = 9 * kInter + 64;   // 32-bit words per activation copy; word 9*512 = the shared gate logit

struct DecodeParams {
  const LayerPtrs* layers;       // device array indexed by layer
  const __nv_bfloat16* x_in;     // [2048] residual stream entering first_layer
  __nv_bfloat16* x_out;          // [2048] residual stream leaving the last layer
  uint32_t* xbuf0;               // [replicas][2048] inter-layer ping-pong, words = tag16 << 16 | bf16
  uint32_t* xbuf1;
  unsigned long long* logits;    // [2][replicas][256] words = tag32 << 32 | FP32 logit bits; the second
                                 // half carries the NEXT layer's router applied to this layer's input
                                 // (the prediction that lets its expert rows be requested early)
  uint32_t* act;                 // [replicas][kDecodeActStride] tagged words (layer tag << 16 | BF16 activation): 8 positions + shared,
                                 // then the shared-expert gate logit as FP32 bits
  unsigned* epoch_base;             // exchange tags used so far (persists across launches)
  int* status;                   // device status word, 0 = healthy
  const float* router_bias;      // [256] or nullptr
  int quant_eighths;
  int speculate;                 // 1: request the predicted experts' rows before the routing is known
  int max_in_flight;             // ring items a block may have requested but not yet received (0: no limit)
  float eps;
  int first_layer;
  int n_layers;
  int expert_lo;                 // experts [expert_lo, expert_hi) live on this GPU
  int expert_hi;
  // expert parallelism: ep_dots[r] is rank r's exchange buffer (own buffer at index `rank`),
  // laid out [2 layer parities][8 rank slots][2048] 64-bit words = tag32 << 32 | FP32 bits
  unsigned long long* ep_dots[8];
  int world;
  int rank;
  // optional tracing: every block stamps %globaltimer at kDecodeTraceSlots points of every layer into
  // timeline[(block * kMaxLayers + layer_ordinal) * kDecodeTraceSlots + k]
  unsigned long long* timeline;
  // optional qualification outputs (last processed layer wins)
  __nv_bfloat16* dbg_h2;
  float* dbg_logits;
  int* dbg_ids;
  float* dbg_scores;
  __nv_bfloat16* dbg_weights;
  __nv_bfloat16* dbg_shared_scaled;
  __nv_bfloat16* dbg_routed;
  float* dbg_slot_dots;          // [8][2048] per-slot down products (FP32) of the locally held experts
};

cudaError_t launch_moe_decode(const DecodeParams& params, int grid_blocks,
                              cudaStream_t stream);

}  // namespace aima
