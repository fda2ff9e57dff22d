// Parameters and launcher of the persistent batch-1 decode kernel.
#pragma once

#include "common.cuh"

namespace aima {

constexpr int kDecodeConsumerWarps = 15;  // + 1 producer = 16 warps, 4 per SM sub-partition
constexpr int kDecodeConsumerThreads = kDecodeConsumerWarps * 32;
constexpr int kDecodeThreads = kDecodeConsumerThreads + 32;  // + producer warp
// Each block owns hidden/grid output elements and stages their down-projection
// rows (8 experts + shared, 1 KB each) in shared memory: at most 14 per block,
// i.e. the grid must have at least ceil(2048 / 14) = 147 blocks.
constexpr int kDecodeMaxRowsPerBlock = 14;
constexpr int kDecodeMinBlocks = (kHidden + kDecodeMaxRowsPerBlock - 1) / kDecodeMaxRowsPerBlock;
constexpr int kDecodeMaxBlocks = kExperts;  // router rows are dealt c, c + grid
constexpr int kDecodeSmemBytes = 221512;
constexpr int kDecodeTraceStamps = 12;

struct DecodeParams {
  const LayerPtrs* layers;       // device array indexed by layer
  const __nv_bfloat16* x_in;     // [2048] residual stream entering first_layer
  __nv_bfloat16* x_out;          // [2048] residual stream leaving the last layer
  __nv_bfloat16* xbuf0;          // [2048] inter-layer ping-pong
  __nv_bfloat16* xbuf1;
  float* logits;                 // [256] scratch
  uint16_t* act;                 // [9 * 512] BF16 activations: 8 ranks + shared
  float* gate_logit;             // [1] shared-expert gate logit (BF16-rounded)
  unsigned long long* bar_counter;  // monotonic grid-barrier arrivals
  unsigned long long* bar_base;     // counter value when this launch starts
  int* status;                   // device status word, 0 = healthy
  const float* router_bias;      // [256] or nullptr
  int quant_eighths;
  float eps;
  int first_layer;
  int n_layers;
  int expert_lo;                 // experts [expert_lo, expert_hi) live on this GPU
  int expert_hi;
  // optional tracing: block 0 stamps %globaltimer at kDecodeTraceStamps points
  // of every layer into timeline[layer_ordinal * kDecodeTraceStamps + k]
  unsigned long long* timeline;
  // optional qualification outputs (last processed layer wins)
  __nv_bfloat16* dbg_h2;
  float* dbg_logits;
  int* dbg_ids;
  float* dbg_scores;
  __nv_bfloat16* dbg_weights;
  __nv_bfloat16* dbg_shared_scaled;
  __nv_bfloat16* dbg_routed;
};

cudaError_t launch_moe_decode(const DecodeParams& params, int grid_blocks,
                              cudaStream_t stream);

}  // namespace aima
