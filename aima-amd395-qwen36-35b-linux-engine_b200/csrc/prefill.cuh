// Prefill MoE half-layer: workspace, per-call description and launcher.
#pragma once

#include "../../include/aima_moe.h"
#include "common.cuh"

namespace aima {

constexpr int kTileRows = 128;      // rows of one grouped-GEMM tile (one expert)
constexpr int kPlanRowsPerWarp = 256;

// Device buffers owned by a handle for prefill calls of up to `capacity` tokens.
struct PrefillWorkspace {
  size_t total_bytes = 0;
  int capacity = 0;
  int sm_count = 0;
  int* status = nullptr;              // device status word shared with the handle
  bool use_simt_gemm = false;         // qualification: CUDA-core products instead of tcgen05
  bool exact_router = false;          // qualification: all 256 logits with the canonical dot
  bool fused_dispatch = true;         // gate_up kernel gathers its rows itself (no materialised copy)
  bool pair_products = false;         // qualification: expert products in the two-SM form (cta_group::2, 256-row tiles)
  uint8_t* base = nullptr;
  // The shared expert does not depend on the routing: it runs on a second stream, forked from and
  // joined to the caller's stream with events, next to the router, the plan and the row gather.
  cudaStream_t side_stream = nullptr;
  cudaEvent_t fork_event = nullptr;     // caller's stream: inputs of this call are ready
  cudaEvent_t router_event = nullptr;   // caller's stream: sigmoid of the shared gate is written
  cudaEvent_t join_event = nullptr;     // side stream: shared expert output is written
  // Expert parallelism: rows arrive (dispatch) and leave (row return) on two more streams, part by
  // part, while the products of another part run on the caller's stream.
  static constexpr int kMaxParts = 8;
  int ep_parts = 1;                               // 1: dispatch, products and return run one after the other
  bool ep_fused_return = true;                    // ep_parts == 1: the down kernel's epilogue stores rows to their owners
  bool ep_fused_dispatch = true;                  // ep_parts == 1: the gate_up kernel gathers its rows from the all-gathered h2
  cudaStream_t inbound_stream = nullptr;
  cudaStream_t outbound_stream = nullptr;
  cudaEvent_t plan_event = nullptr;               // caller's stream: the plan is written
  cudaEvent_t published_event = nullptr;          // inbound stream: this rank's h2 rows are stored on every GPU
  cudaEvent_t gathered_event[kMaxParts] = {};     // inbound stream: rows of part k are here
  cudaEvent_t computed_event[kMaxParts] = {};     // caller's stream: products of part k are written
  cudaEvent_t returned_event = nullptr;           // outbound stream: all rows are stored and flagged
  // router outputs
  int32_t* topk_ids = nullptr;        // [T, 8]
  float* topk_scores = nullptr;       // [T, 8]
  float* topk_weights = nullptr;      // [T, 8] BF16-rounded, stored as FP32
  float* shared_sigmoid = nullptr;    // [T]    bf16(sigmoid(bf16 gate logit)) as FP32
  float* approx_logits = nullptr;     // [T, 256] tensor-core router logits (candidate filter only)
  int32_t* router_stats = nullptr;    // [5] candidates recomputed exactly, tokens routed, tokens whose candidates broke the
                                      //     filter's bound (recomputed in full), tokens audited, audit mismatches
  int router_audit_stride = 0;        // qualification: every n-th token is also routed from all 256 canonical logits
  // dispatch plan
  int32_t* unit_counts = nullptr;     // [units, 256] per-warp-unit histogram / prefix
  int32_t* expert_counts = nullptr;   // [256]
  int32_t* expert_offsets = nullptr;  // [257]
  int32_t* sorted_rows = nullptr;     // [8T]  flat (token*8+slot) rows grouped by expert
  int32_t* row_position = nullptr;    // [8T]  inverse of sorted_rows
  int32_t* tile_expert = nullptr;     // [max_tiles]
  int32_t* tile_row0 = nullptr;       // [max_tiles]
  int32_t* tile_rows = nullptr;       // [max_tiles]
  int32_t* tile_count = nullptr;      // [1]
  int32_t* padded_rows = nullptr;     // [1] block-32 padded row count of the reference plan
  // activations
  __nv_bfloat16* gathered = nullptr;      // [8T, 2048] h2 rows in sorted order
  __nv_bfloat16* expert_act = nullptr;    // [8T, 512]
  __nv_bfloat16* expert_down = nullptr;   // [8T, 2048] weighted, sorted order
  __nv_bfloat16* shared_act = nullptr;    // [T, 512]
  __nv_bfloat16* shared_scaled = nullptr; // [T, 2048]
  // layer-stack buffers
  __nv_bfloat16* stack_x0 = nullptr;      // [T, 2048]
  __nv_bfloat16* stack_x1 = nullptr;
  __nv_bfloat16* stack_h2 = nullptr;
};

// Exchange region of one GPU for expert-parallel prefill (inside its IPC-shared allocation).
struct EpPrefillLayout {
  size_t off_flags_routing;   // u32[8]  rank q has published its routing for epoch e
  size_t off_flags_returned;  // u32[8]  rank q has returned all rows it computed for epoch e
  size_t off_ids;             // i32 [T * 8]  routing ids of all ranks, rank-major
  size_t off_weights;         // f32 [T * 8]
  size_t off_h2;              // bf16 [T, 2048] the tokens of all ranks, rank-major; every rank stores its rows here on every GPU
  size_t off_return;          // bf16 [T_loc * 8, 2048] weighted expert outputs of this rank's tokens
  size_t bytes;
};

struct EpPrefill {
  int world = 1;
  int rank = 0;
  uint8_t* peers[8] = {};     // every rank's region (own included)
  EpPrefillLayout layout{};
  unsigned epoch = 0;         // calls so far; all ranks call in lockstep
  // optional stage timing (tracing): events at the 8 stage boundaries of the last call
  cudaEvent_t stage_events[8] = {};
  bool trace = false;
};
constexpr int kEpPrefillStages = 7;   // route, routing exchange, plan, dispatch, experts, return, shared+wait+combine

struct PrefillCall {
  LayerPtrs layer;
  const void* h2;
  const void* residual;
  void* out;
  int tokens;
  int experts_local;             // experts held in the bound expert tensors
  const float* router_row_norms; // [256] Euclidean norms of the router rows (certified filter)
  const float* router_bias;
  int quant_eighths;
  const aima_moe_debug_views* debug;
  // qualification: routing supplied by the harness instead of the router's (ids i32 [T, 8], weights BF16 [T, 8])
  const int32_t* forced_ids = nullptr;
  const void* forced_weights = nullptr;
  // optional fused exit: RMSNorm of the layer output with this weight (the next layer's input norm)
  const void* next_norm_weight = nullptr;
  void* next_norm_out = nullptr;
  float eps = 1.0e-6f;
};

size_t prefill_workspace_bytes(uint32_t capacity_tokens);
int prefill_workspace_allocate(PrefillWorkspace* workspace, uint32_t capacity_tokens,
                               int sm_count, char* error, size_t error_bytes);
void prefill_workspace_free(PrefillWorkspace* workspace);

// Euclidean norm of each of the 256 router rows (FP32), computed once per layer at bind time.
cudaError_t launch_router_row_norms(const __nv_bfloat16* router, float* norms, cudaStream_t stream);

// Enqueues the whole half-layer on `stream`; `launches` receives the number of
// kernels enqueued.  Returns an AIMA_MOE_* status.
int prefill_layer_launch(PrefillWorkspace* workspace, const PrefillCall& call,
                         cudaStream_t stream, int* launches, char* error,
                         size_t error_bytes);

size_t ep_prefill_region_bytes(int capacity_tokens, int world, EpPrefillLayout* layout);

// Expert-parallel variant: call.tokens = this rank's tokens; all ranks call in lockstep.
int prefill_layer_launch_ep(PrefillWorkspace* workspace, const PrefillCall& call, EpPrefill* ep,
                            cudaStream_t stream, int* launches, char* error, size_t error_bytes);

inline int max_tiles_for(int tokens) {
  return tokens * kTopK / kTileRows + kExperts;
}

}  // namespace aima
