// Grouped (per-expert) BF16 products of the prefill path.
//
// A problem is a list of row tiles; tile t multiplies rows
// [tile_row0[t], tile_row0[t] + tile_rows[t]) of A by the weight matrix of
// expert tile_expert[t] (B is [n, k] row-major, i.e. C = A . B^T, FP32
// accumulation).  With tile_expert == nullptr the product is dense over
// `dense_rows` rows in tiles of kTileRows.
//
// Epilogues (rounding points of native/src/native_moe_prefill.hip.cpp):
//   kGemmExpertGateUp  act = bf16(f32(bf16(silu(bf16 g))) * bf16 u)      (:384-402)
//   kGemmSharedGateUp  act = bf16(silu(bf16 g) * bf16 u)                 (:210-219)
//   kGemmExpertDown    out = bf16(acc * routing_weight[flat row])        (fused_moe down,
//                            MUL_ROUTED_WEIGHT; manifest.json:4672-4689)
//   kGemmSharedDown    out = bf16(bf16(sigmoid gate)[row] * bf16(acc))   (:221-232)
// In the two gate_up modes column i of the output pairs weight rows i (gate) and
// n + i (up; b1 when it is a separate tensor).
#pragma once

#include "common.cuh"

namespace aima {

constexpr int kTileRowsSimt = 128;  // must equal kTileRows of the dispatch plan

enum GemmMode {
  kGemmExpertGateUp = 0,
  kGemmSharedGateUp = 1,
  kGemmExpertDown = 2,
  kGemmSharedDown = 3,
  kGemmPlain = 4,     // out = bf16(acc): the contract of Bf16GemmPlan::launch
                      // (native/src/bf16_gemm.hip.cpp:220-234), dense rows only
  kGemmPlainF32 = 5,  // out = acc as FP32 into c_f32 (approximate router logits)
};

struct GroupedGemm {
  const int32_t* tile_expert;
  const int32_t* tile_row0;
  const int32_t* tile_rows;
  const int32_t* tile_count;   // device scalar; nullptr in dense mode
  int expert_base;             // first expert held in b0 (tile_expert holds global ids)
  int max_tiles;               // launch bound on the tile count
  int dense_rows;
  const __nv_bfloat16* a;      // [rows, k]
  int lda;
  // kGemmExpertGateUp on the tensor cores only: when non-null, tile row r is row
  // (sorted_rows[row] >> 3) of this [tokens, k] matrix, gathered straight into shared memory
  // (no materialised copy of the routed rows); `a` is then unused
  const __nv_bfloat16* gather_src;
  int k;
  const __nv_bfloat16* b0;     // gate (or only) weight matrix / expert slab
  const __nv_bfloat16* b1;     // separate "up" matrix (shared expert) or nullptr
  size_t b_expert_stride;      // elements between experts in b0
  int n;                       // output columns
  __nv_bfloat16* c;            // [rows, n]
  float* c_f32;                // FP32 output of kGemmPlainF32
  int ldc;
  const float* row_scale;      // routing weights [T*8] or sigmoid gate [T]
  const int32_t* sorted_rows;  // flat routed row of each sorted position
  // tensor-core kernel only: this launch covers tiles [n * part / parts, n * (part + 1) / parts) of the
  // n tiles of the plan (parts <= 1: all of them), so that copies for one part overlap products of another
  int part;
  int parts;
  // kGemmExpertDown on the tensor cores, expert parallelism: when scatter_tokens_per_rank > 0 the weighted row
  // of flat routed row f = sorted_rows[row] is not stored to c but straight to the GPU that owns its token,
  // at row f - owner * 8 * scatter_tokens_per_rank of the [tokens_per_rank * 8, n] matrix at
  // scatter_region[owner] + scatter_offset (plain peer stores from the epilogue, no copy kernel afterwards)
  uint8_t* scatter_region[8];
  size_t scatter_offset;
  int scatter_tokens_per_rank;
};

// What the tensor-core launcher needs beyond the problem itself.
struct TcExtra {
  int* status;          // device status word for bounded-wait expiry
  int sm_count;         // persistent grid size
  uint64_t a_rows;      // rows of the A allocation (TMA bounds; reads beyond are zero-filled)
  int experts_in_b;     // experts held in b0 (expert modes), else 1
  bool pair = false;    // expert modes: two-SM form; the plan's tiles then hold up to 256 rows
};

// tcgen05 / TMEM / TMA implementation (grouped_gemm_tc.cu).
cudaError_t launch_grouped_gemm_tc(GemmMode mode, const GroupedGemm& problem,
                                   const TcExtra& extra, cudaStream_t stream);

// CUDA-core implementation kept as an on-device cross-check of the tensor-core
// kernel (selected per call by the qualification flag).
cudaError_t launch_grouped_gemm_simt(GemmMode mode, const GroupedGemm& problem,
                                     cudaStream_t stream);

}  // namespace aima
