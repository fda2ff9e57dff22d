// LM head with a certified top-1 (see lm_head.cu).
#pragma once

#include "../../include/aima_moe.h"
#include "common.cuh"

namespace aima {

struct LmHeadBuffers {
  int8_t* q_weight;                 // [rows, 2048]
  float* scales;                    // [rows]
  float* residual_l2;               // [rows]
  aima_moe_lm_head_result* wire;    // device copy of the result
  float* partial;                   // [256] per-block maxima of the lower bounds
  uint32_t* candidate_ids;          // [AIMA_MOE_LM_HEAD_CANDIDATES]
};

cudaError_t lm_head_quantize(const void* weight, int rows, int8_t* q_weight, float* scales, float* residual_l2,
                             cudaStream_t stream);

// Enqueues the scan, the bounds, the candidate collection and the exact candidate logits with their arg-max.
cudaError_t lm_head_certify(const LmHeadBuffers& buffers, const void* weight, const void* hidden, float* logits,
                            int rows, int sm_count, cudaStream_t stream, int* launches);

}  // namespace aima
