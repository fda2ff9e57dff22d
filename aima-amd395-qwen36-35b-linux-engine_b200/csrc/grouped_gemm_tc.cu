// Grouped BF16 products on the 5th-generation tensor cores (tcgen05 + TMEM),
// operands staged by TMA, for the prefill expert and shared-expert products.
//
// Replaces the two fused_moe_kernel launches of the reference prefill path
// (native/aot/gfx1151/q8192-output2/manifest.json:1398-1415, 4672-4689; launched
// at native/src/native_moe_prefill.hip.cpp:862-876), expert_silu_multiply_kernel
// (:384-402), and the five hipBLASLt plans of the shared expert with their
// pointwise kernels (:790-826) -- the epilogues are fused.
//
// Work unit = one 128-row tile of one expert x one 256-wide slice of the output
// columns.  D[128, 256] (FP32) lives in tensor memory, two buffers of 256
// columns, so the epilogue of a unit overlaps the main loop of the next.
//   warp 0   TMA producer: per 64-wide K block one 128x64 tile of A and two
//            128x64 tiles of B into a 4-stage shared-memory ring (128-byte swizzle)
//   warp 1   one thread issues tcgen05.mma (M128 N256 K16, 4 per K block) and
//            commits to the ring's "empty" barriers / the accumulator's "full" barrier
//   warp 2   allocates and frees the 512 tensor-memory columns
//   warps 2-3 with fused dispatch (gate_up only): gather the tile's 128 activation rows BY TOKEN
//            INDEX with 16-byte cp.async copies that arrive on the stage's barrier when complete
//   warps 4-11 epilogue (two per quarter of the TMEM lanes, half of the columns each): tcgen05.ld 32 rows x 32 columns per warp, SwiGLU or
//            scaling; the BF16 results of 64 output columns are turned in shared memory so that
//            every store instruction writes whole 128-byte pieces of four rows (a thread storing
//            its own row would touch 32 different lines per instruction)
// Every mbarrier wait is bounded; on expiry the block sets the status word,
// stops issuing, waits for its copies in flight, frees tensor memory and returns.
#include "grouped_gemm.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <cudaTypedefs.h>

namespace aima {
namespace {

constexpr int kBM = 128;           // rows per tile (= kTileRows of the plan)
constexpr int kBN = 256;           // accumulator columns per unit
constexpr int kBK = 64;            // K elements per stage: 128 bytes = one swizzle row
constexpr int kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kStageABytes = kBM * kBK * 2;        // 16 KB
constexpr int kStageBBytes = kBN * kBK * 2;        // 32 KB
constexpr int kStageBytes = kStageABytes + kStageBBytes;
constexpr int kEpilogueWarps = 8;   // two per quarter of the 128 TMEM lanes, each taking half of the columns
constexpr int kTcThreads = (4 + kEpilogueWarps) * 32;
constexpr int kTmemColumns = 512;
constexpr int kStoreStageBytes = 32 * 128;          // per epilogue warp: 32 rows x 64 BF16 outputs
constexpr int kTcSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ +
                             kEpilogueWarps * kStoreStageBytes;

struct TcMaps {
  CUtensorMap a;    // [rows, k]      box 64 x 128
  CUtensorMap b0;   // gate half / only weight matrix, [n_rows, k]
  CUtensorMap b1;   // up half (may equal b0)
};

struct TcProblem {
  GroupedGemm g;
  int n_chunks;           // output column slices of kBN accumulator columns
  int b_rows_per_expert;  // rows between experts in b0 / b1
  int up_row_offset;      // row offset of the "up" half inside an expert (gate_up modes)
  int n_valid;            // valid output columns (plain mode masks beyond)
  int a_rows;             // rows of the A tensor (fused dispatch: first out-of-range row index)
  int* status;            // device status word
};

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
constexpr int kGatherThreads = 64;     // warps 2 and 3
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src) : "memory");
}
// the barrier receives one arrival (already part of its expected count) once all cp.async copies this
// thread has issued so far are complete
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               :: "r"(smem_dst), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes
// (64 BF16) with the 128-byte swizzle TMA applies: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);          // start address
  desc |= static_cast<uint64_t>(1) << 16;                               // leading byte offset (unused)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;                       // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;                               // descriptor version (sm_100)
  desc |= static_cast<uint64_t>(2) << 61;                               // SWIZZLE_128B
  return desc;
}

// Instruction descriptor: D = F32, A = B = BF16, both K-major, M = 128, N = 256.
constexpr uint32_t kInstrDesc =
    (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kBN >> 3) << 17) |
    (static_cast<uint32_t>(kBM >> 4) << 24);

// 32 results of this thread's row into half `half` (0/1) of the warp's 32 x 128-byte staging
// tile; 16-byte pieces are XOR-swizzled by the row so that neither side has bank conflicts.
__device__ __forceinline__ void stage_32(uint8_t* stage, int lane, int half, const float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 w;
    w.x = static_cast<uint32_t>(float_to_bf16_bits(v[8 * i + 0])) | (static_cast<uint32_t>(float_to_bf16_bits(v[8 * i + 1])) << 16);
    w.y = static_cast<uint32_t>(float_to_bf16_bits(v[8 * i + 2])) | (static_cast<uint32_t>(float_to_bf16_bits(v[8 * i + 3])) << 16);
    w.z = static_cast<uint32_t>(float_to_bf16_bits(v[8 * i + 4])) | (static_cast<uint32_t>(float_to_bf16_bits(v[8 * i + 5])) << 16);
    w.w = static_cast<uint32_t>(float_to_bf16_bits(v[8 * i + 6])) | (static_cast<uint32_t>(float_to_bf16_bits(v[8 * i + 7])) << 16);
    const int piece = (4 * half + i) ^ (lane & 7);
    *reinterpret_cast<uint4*>(stage + lane * 128 + piece * 16) = w;
  }
}

// The staged 32 x 64 tile to global memory: instruction i writes rows 4i .. 4i+3, eight lanes per
// row.  dst = first row of the warp's 32, first of the 64 columns; rows_ok = valid rows of the 32;
// cols_ok = valid columns of the 64 (a multiple of 8).
__device__ __forceinline__ void store_staged(const uint8_t* stage, int lane, __nv_bfloat16* dst, size_t ldc,
                                             int rows_ok, int cols_ok) {
  __syncwarp();
  const int piece = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = 4 * i + (lane >> 3);
    const uint4 w = *reinterpret_cast<const uint4*>(stage + row * 128 + ((piece ^ (row & 7)) * 16));
    if (row < rows_ok && piece * 8 < cols_ok)
      *reinterpret_cast<uint4*>(dst + static_cast<size_t>(row) * ldc + piece * 8) = w;
  }
  __syncwarp();
}


// The same with one destination per row: rows[i] is the address of the first of the 64 columns in the row
// instruction i writes for this lane (row 4 i + lane / 8 of the warp's 32), nullptr for a row past the tile's end.
__device__ __forceinline__ void store_staged_rows(const uint8_t* stage, int lane, __nv_bfloat16* const* rows, int cols_ok) {
  __syncwarp();
  const int piece = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = 4 * i + (lane >> 3);
    const uint4 w = *reinterpret_cast<const uint4*>(stage + row * 128 + ((piece ^ (row & 7)) * 16));
    if (rows[i] != nullptr && piece * 8 < cols_ok) *reinterpret_cast<uint4*>(rows[i] + piece * 8) = w;
  }
  __syncwarp();
}

// One epilogue warp drains its part of a 128-row x 256-column FP32 accumulator: TMEM lanes
// 32 ew .. 32 ew + 31 (rows row0 + 32 ew ... of the output), half `eh` of the unit's columns.
template <int MODE>
__device__ __forceinline__ void drain_accumulator(const GroupedGemm& g, const TcProblem& pb, uint32_t tmem_base,
                                                  int buf, int ew, int eh, int lane, uint8_t* stage, int chunk,
                                                  int row0, int rows) {
  constexpr bool kDual = (MODE == kGemmExpertGateUp || MODE == kGemmSharedGateUp);
  const int r = ew * 32 + lane;                // row inside the tile
  const bool row_ok = r < rows;
  const int row = row0 + r;
  const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + static_cast<uint32_t>(buf * kBN);
  const int rows_ok = min(32, rows - ew * 32);           // valid rows among this warp's 32 (may be <= 0)
  if (kDual) {
    // columns [0,128) gate, [128,256) up  ->  128 activations per row, stored 64 at a time
    __nv_bfloat16* dst = g.c + static_cast<size_t>(row0 + ew * 32) * g.ldc + chunk * (kBN / 2);
#pragma unroll 1
    for (int c0 = eh * (kBN / 4); c0 < (eh + 1) * (kBN / 4); c0 += 64) {
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t gr[32], ur[32];
        tmem_ld32(taddr + c0 + 32 * half, gr);
        tmem_ld32(taddr + kBN / 2 + c0 + 32 * half, ur);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float gate = round_bf16(__uint_as_float(gr[j]));
          const float up = round_bf16(__uint_as_float(ur[j]));
          const float s = det_silu(gate);
          v[j] = (MODE == kGemmExpertGateUp) ? __fmul_rn(round_bf16(s), up) : __fmul_rn(s, up);
        }
        stage_32(stage, lane, half, v);
      }
      store_staged(stage, lane, dst + c0, static_cast<size_t>(g.ldc), rows_ok, 64);
    }
  } else if (MODE != kGemmPlainF32) {
    float scale = 1.0f;
    if (row_ok) {
      if (MODE == kGemmExpertDown) scale = g.row_scale[g.sorted_rows[row]];
      if (MODE == kGemmSharedDown) scale = g.row_scale[row];
    }
    const int col_base = chunk * kBN;
    __nv_bfloat16* dst = g.c + static_cast<size_t>(row0 + ew * 32) * g.ldc + col_base;
    const bool scatter = MODE == kGemmExpertDown && g.scatter_tokens_per_rank > 0;
    __nv_bfloat16* scatter_rows[8];
    if (scatter) {
      // where the eight rows this lane stores live: on the GPU that owns the row's token
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + (lane >> 3);
        scatter_rows[i] = nullptr;
        if (rr < rows_ok) {
          const int flat = g.sorted_rows[row0 + ew * 32 + rr];
          const int owner = (flat >> 3) / g.scatter_tokens_per_rank;
          const int local_flat = flat - owner * g.scatter_tokens_per_rank * 8;
          scatter_rows[i] = reinterpret_cast<__nv_bfloat16*>(g.scatter_region[owner] + g.scatter_offset) +
                            static_cast<size_t>(local_flat) * g.ldc + col_base;
        }
      }
    }
#pragma unroll 1
    for (int c0 = eh * (kBN / 2); c0 < (eh + 1) * (kBN / 2); c0 += 64) {
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t ar[32];
        tmem_ld32(taddr + c0 + 32 * half, ar);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float acc = __uint_as_float(ar[j]);
          if (MODE == kGemmExpertDown) v[j] = __fmul_rn(acc, scale);
          else if (MODE == kGemmSharedDown) v[j] = __fmul_rn(scale, round_bf16(acc));
          else v[j] = acc;
        }
        stage_32(stage, lane, half, v);
      }
      const int cols_ok = max(0, min(64, pb.n_valid - col_base - c0));
      if (scatter) {
        __nv_bfloat16* at[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) at[i] = scatter_rows[i] != nullptr ? scatter_rows[i] + c0 : nullptr;
        store_staged_rows(stage, lane, at, cols_ok);
      } else {
        store_staged(stage, lane, dst + c0, static_cast<size_t>(g.ldc), rows_ok, cols_ok);
      }
    }
  } else {
    // FP32 output (approximate router logits): every thread stores its own row
    const int col_base = chunk * kBN;
#pragma unroll 1
    for (int c0 = eh * (kBN / 2); c0 < (eh + 1) * (kBN / 2); c0 += 32) {
      uint32_t ar[32];
      tmem_ld32(taddr + c0, ar);
      tmem_ld_wait();
      if (row_ok) {
        float4* out = reinterpret_cast<float4*>(g.c_f32 + static_cast<size_t>(row) * g.ldc + col_base + c0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (col_base + c0 + 4 * j + 4 <= pb.n_valid)
            out[j] = make_float4(__uint_as_float(ar[4 * j]), __uint_as_float(ar[4 * j + 1]),
                                 __uint_as_float(ar[4 * j + 2]), __uint_as_float(ar[4 * j + 3]));
        }
      }
    }
  }
}

template <int MODE, bool kGather = false>
__global__ void __launch_bounds__(kTcThreads, 1)
grouped_gemm_tc_kernel(const __grid_constant__ TcMaps maps, const TcProblem pb) {
  constexpr bool kDual = (MODE == kGemmExpertGateUp || MODE == kGemmSharedGateUp);
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the swizzled descriptors assume base offset 0
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + kStages * kStageBytes + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kStages * kStageBytes + 8 * (2 * kStages + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const GroupedGemm& g = pb.g;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), kGather ? 1 + kGatherThreads : 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), kEpilogueWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 2) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemColumns);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Programmatic dependent launch: the kernel is launched with stream serialisation relaxed, so its
  // blocks may become resident -- and run the set-up above (barriers, TMEM) -- while the kernel
  // before it in the stream is still draining.  Nothing above reads or writes global memory;
  // everything below does, so this is where the kernel waits for its predecessor to complete and
  // for that kernel's writes to be visible.  The kernel after this one may be scheduled likewise.
  pdl_enter();

  const int n_tiles_all = g.tile_count != nullptr ? *g.tile_count : g.max_tiles;
  const int parts = g.parts > 1 ? g.parts : 1;
  const int tile_lo = static_cast<int>(static_cast<long long>(n_tiles_all) * g.part / parts);
  const int tile_hi = static_cast<int>(static_cast<long long>(n_tiles_all) * (g.part + 1) / parts);
  // a bounded wait that ran out earlier in this call (a peer that never answered, a barrier of a kernel before
  // this one) leaves a status: nothing that follows can be right, so the products are skipped rather than run on
  // incomplete data until the host reads the status
  // (one thread samples it for the block, so that all warp roles see the same verdict)
  volatile int* poison_slot = abort_flag + 1;
  if (threadIdx.x == 0) *poison_slot = *reinterpret_cast<volatile const int*>(pb.status);
  __syncthreads();
  const bool poisoned = *poison_slot != 0;
  const int total_units = poisoned ? 0 : (tile_hi - tile_lo) * pb.n_chunks;
  const int k_blocks = g.k / kBK;

  auto unit_tile = [&](int unit, int& tile, int& chunk, int& expert, int& row0, int& rows) {
    tile = unit / pb.n_chunks;
    chunk = unit - tile * pb.n_chunks;
    tile += tile_lo;
    if (g.tile_expert != nullptr) {
      expert = g.tile_expert[tile] - g.expert_base;
      row0 = g.tile_row0[tile];
      rows = g.tile_rows[tile];
    } else {
      expert = 0;
      row0 = tile * kBM;
      rows = min(kBM, g.dense_rows - row0);
    }
  };
  auto timeout = [&]() {
    atomicCAS(pb.status, 0, kStatusTimeoutMbarrier);
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool alive = true;
      for (int unit = blockIdx.x; unit < total_units && alive; unit += gridDim.x) {
        int tile, chunk, expert, row0, rows;
        unit_tile(unit, tile, chunk, expert, row0, rows);
        int b0_row, b1_row;
        if (kDual) {
          b0_row = expert * pb.b_rows_per_expert + chunk * (kBN / 2);
          b1_row = expert * pb.b_rows_per_expert + pb.up_row_offset + chunk * (kBN / 2);
        } else {
          b0_row = expert * pb.b_rows_per_expert + chunk * kBN;
          b1_row = b0_row + kBN / 2;
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kStageABytes;
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag)) { alive = false; timeout(); break; }
          mbar_arrive_expect_tx(full_bar(stage), kGather ? kStageBBytes : kStageBytes);
          if (!kGather) tma_load_2d(a_dst, &maps.a, kb * kBK, row0, full_bar(stage));
          tma_load_2d(b_dst, &maps.b0, kb * kBK, b0_row, full_bar(stage));
          tma_load_2d(b_dst + kStageBBytes / 2, kDual ? &maps.b1 : &maps.b0, kb * kBK, b1_row, full_bar(stage));
          ++issued;
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      // drain on abort: wait (bounded) for the stages whose copies are still in flight
      if (*abort_flag != 0) {
        volatile int ignore = 0;
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < min(issued, kStages); ++i) {
          if (--s < 0) { s = kStages - 1; ph ^= 1u; }
          mbar_wait_bounded(full_bar(s), ph, &ignore);
        }
      }
    }
  } else if (kGather && (warp == 2 || warp == 3)) {
    // ------------------------------ A-row gather -------------------------------
    // Eight neighbouring threads copy the eight 16-byte pieces of one row per K block (a warp
    // instruction then touches four 128-byte lines, not 32): thread t owns piece t % 8 of rows
    // t / 8 + 8 j, j = 0 .. 15, fetched by token index; piece c of row r goes to piece position
    // c ^ (r & 7) (the 128-byte swizzle).  The copies are asynchronous and the thread never waits for
    // them: an arrive-on-completion on the stage's "full" barrier (already counted in the barrier's
    // arrival count) follows each batch, so the only wait is for a free stage and up to kStages
    // batches per thread stay in flight.
    const int lt = (warp - 2) * 32 + lane;
    const int piece = lt & 7;
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int unit = blockIdx.x; unit < total_units && alive; unit += gridDim.x) {
      int tile, chunk, expert, row0, rows;
      unit_tile(unit, tile, chunk, expert, row0, rows);
      int source[16];            // element offset of this thread's piece in each of its 16 rows
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int r = (lt >> 3) + 8 * j;
        const int token = g.sorted_rows[row0 + min(r, rows - 1)] >> 3;   // rows past the tile's end repeat its last row
        source[j] = token * g.lda + piece * 8;
      }
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag)) { alive = false; timeout(); break; }
        const uint32_t base = smem_base + stage * kStageBytes;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int r = (lt >> 3) + 8 * j;
          cp_async_16(base + r * 128 + ((piece ^ (r & 7)) << 4), g.gather_src + source[j] + kb * kBK);
        }
        cp_async_arrive_noinc(full_bar(stage));
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    cp_async_wait_all();     // nothing of this thread's may be in flight when the block exits
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool alive = true;
      for (int unit = blockIdx.x; unit < total_units && alive; unit += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        // the epilogue must have drained this accumulator buffer (first use: free)
        if (!mbar_wait_bounded(tempty_bar(buf), (use & 1u) ^ 1u, abort_flag)) { alive = false; timeout(); break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kBN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag)) { alive = false; timeout(); break; }
          if (kGather) fence_async_proxy();     // rows written by cp.async are read through the async proxy
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * kStageBytes;
          const uint32_t b_addr = a_addr + kStageABytes;
          const uint64_t adesc = smem_desc_k_major_sw128(a_addr);
          const uint64_t bdesc = smem_desc_k_major_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // advancing 16 elements (32 bytes) along K inside the swizzled row
            umma_bf16(tmem_d, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2),
                      kInstrDesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));      // frees the stage when the MMAs above retire
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (alive) umma_commit(tfull_bar(buf));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue ----------------------------------
    const int ew = (warp - 4) & 3;                 // TMEM lanes 32 ew .. 32 ew + 31 (a warp reaches the quarter warp % 4)
    const int eh = (warp - 4) >> 2;                // which half of the unit's columns this warp drains
    int local = 0;
    bool alive = true;
    for (int unit = blockIdx.x; unit < total_units && alive; unit += gridDim.x, ++local) {
      int tile, chunk, expert, row0, rows;
      unit_tile(unit, tile, chunk, expert, row0, rows);
      const int buf = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      if (!mbar_wait_bounded(tfull_bar(buf), use & 1u, abort_flag)) { alive = false; if (lane == 0) timeout(); break; }
      tc_fence_after();
      drain_accumulator<MODE>(g, pb, tmem_base, buf, ew, eh, lane,
                              smem_gen + kStages * kStageBytes + 256 + (warp - 4) * kStoreStageBytes, chunk, row0, rows);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, kTmemColumns);
}

// ---------------------------------------------------------------------------
// Two-SM form.  A pair of blocks (a cluster of two) works on one tile of up to 256 rows of one expert x
// 256 accumulator columns with tcgen05.mma.cta_group::2: block r of the pair holds rows 128 r .. 128 r + 127
// of A and one half of B (128 weight rows) per K block, 32 KB per stage instead of 48, so six stages fit
// and every weight byte enters shared memory once per 256 rows instead of once per 128.  The leader (block 0
// of the pair) issues the MMAs for both; each block drains the 128 accumulator rows in its own tensor memory.
//
//   full[s]    leader only.  Completed by the TMA loads of BOTH blocks (cta_group::2 loads signal the
//              leader's barrier), by the leader's gather threads and by the peer's forwarder.
//   gdone[s]   peer only, gather mode: its gather threads' copies of a stage have landed; its forwarder
//              (the peer's otherwise idle MMA warp) then arrives on the leader's full[s].
//   empty[s]   both blocks: the MMAs reading stage s have retired (tcgen05.commit, multicast to the pair).
//   tfull[b]   both blocks: accumulator b is complete (commit, multicast).
//   tempty[b]  leader only: the eight epilogue warps of each block have drained accumulator b.
// No load uses cluster multicast: each block fetches its own operands.
// ---------------------------------------------------------------------------
constexpr int kStages2 = 6;
constexpr int kStage2ABytes = kBM * kBK * 2;              // 16 KB: this block's 128 rows of A
constexpr int kStage2BBytes = (kBN / 2) * kBK * 2;        // 16 KB: this block's half of B
constexpr int kStage2Bytes = kStage2ABytes + kStage2BBytes;
constexpr int kTc2BarrierBytes = 512;
constexpr int kTc2SmemBytes = kStages2 * kStage2Bytes + 1024 /*alignment slack*/ + kTc2BarrierBytes +
                              kEpilogueWarps * kStoreStageBytes;
static_assert(kTc2SmemBytes <= 227 * 1024, "two-SM product kernel exceeds 227 KB of shared memory");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in block `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
// TMA tile load of one block of the pair; the bytes are accounted on the LEADER's barrier
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               :: "r"(smem_dst), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  const uint32_t zero = 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}
// arrives on the barrier at the same shared-memory offset in both blocks of the pair once the MMAs issued so far retire
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               :: "r"(bar), "h"(both) : "memory");
}

// D = F32, A = B = BF16, both K-major, M = 256 (128 rows per block), N = 256.
constexpr uint32_t kInstrDesc2 =
    (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kBN >> 3) << 17) |
    (static_cast<uint32_t>((2 * kBM) >> 4) << 24);

template <int MODE, bool kGather>
__global__ void __launch_bounds__(kTcThreads, 1)
grouped_gemm_tc2_kernel(const __grid_constant__ TcMaps maps, const TcProblem pb) {
  static_assert(MODE == kGemmExpertGateUp || MODE == kGemmExpertDown, "two-SM form: the expert products");
  constexpr bool kDual = (MODE == kGemmExpertGateUp);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kStages2 * kStage2Bytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages2 + s); };
  auto gdone_bar = [&](int s) { return bar_base + 8u * (2 * kStages2 + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (3 * kStages2 + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (3 * kStages2 + 2 + b); };
  uint8_t* tail = smem_gen + kStages2 * kStage2Bytes + 8 * (3 * kStages2 + 4);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);
  uint8_t* store_stage = smem_gen + kStages2 * kStage2Bytes + kTc2BarrierBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: leader of the pair
  const bool leader = rank == 0;
  const GroupedGemm& g = pb.g;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(full_bar(s), kGather ? 1 + kGatherThreads + 1 : 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(gdone_bar(s), kGatherThreads);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 2 * kEpilogueWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 2) tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemColumns);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // both blocks' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_enter();

  const int n_tiles = g.tile_count != nullptr ? *g.tile_count : g.max_tiles;
  // as in the one-SM kernel; the leader samples the status for the pair
  volatile int* poison_slot = abort_flag + 1;
  if (threadIdx.x == 0 && leader) {
    const int seen = *reinterpret_cast<volatile const int*>(pb.status);
    *poison_slot = seen;
    asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(map_to_rank(smem_u32(const_cast<int*>(poison_slot)), 1)), "r"(seen) : "memory");
  }
  __syncthreads();
  cluster_sync_all();
  const bool poisoned = *poison_slot != 0;
  const int total_units = poisoned ? 0 : n_tiles * pb.n_chunks;
  const int n_pairs = gridDim.x >> 1;
  const int pair = blockIdx.x >> 1;
  const int k_blocks = g.k / kBK;

  // unit -> the tile's expert, this block's first row, its number of valid rows (0 .. 128) and the tile's last row
  auto unit_tile = [&](int unit, int& chunk, int& expert, int& row0, int& rows, int& tile_last) {
    const int tile = unit / pb.n_chunks;
    chunk = unit - tile * pb.n_chunks;
    expert = g.tile_expert[tile] - g.expert_base;
    const int tile_rows = g.tile_rows[tile];
    const int tile_row0 = g.tile_row0[tile];
    tile_last = tile_row0 + tile_rows - 1;
    row0 = tile_row0 + static_cast<int>(rank) * kBM;
    rows = max(0, min(kBM, tile_rows - static_cast<int>(rank) * kBM));
  };
  auto timeout = [&]() { atomicCAS(pb.status, 0, kStatusTimeoutMbarrier); };

  if (warp == 0) {
    // ------------------------------ TMA producer (both blocks) -----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int unit = pair; unit < total_units && alive; unit += n_pairs) {
        int chunk, expert, row0, rows, tile_last;
        unit_tile(unit, chunk, expert, row0, rows, tile_last);
        // this block's half of B: gate_up -- the leader takes the 128 gate rows of the chunk, the peer the 128
        // up rows; down -- rows 128 r .. of the chunk's 256 output columns
        const int b_row = kDual ? expert * pb.b_rows_per_expert + static_cast<int>(rank) * pb.up_row_offset + chunk * (kBN / 2)
                                : expert * pb.b_rows_per_expert + chunk * kBN + static_cast<int>(rank) * (kBN / 2);
        for (int kb = 0; kb < k_blocks; ++kb) {
          const uint32_t a_dst = smem_base + stage * kStage2Bytes;
          const uint32_t b_dst = a_dst + kStage2ABytes;
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag)) { alive = false; timeout(); break; }
          const uint32_t leader_full = map_to_rank(full_bar(stage), 0);
          if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * (kGather ? kStage2BBytes : kStage2Bytes));
          if (!kGather) tma_load_2d_pair(a_dst, &maps.a, kb * kBK, row0, leader_full);
          tma_load_2d_pair(b_dst, &maps.b0, kb * kBK, b_row, leader_full);
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (kGather && (warp == 2 || warp == 3)) {
    // ------------------------------ A-row gather (both blocks) -----------------
    const int lt = (warp - 2) * 32 + lane;
    const int piece = lt & 7;
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int unit = pair; unit < total_units && alive; unit += n_pairs) {
      int chunk, expert, row0, rows, tile_last;
      unit_tile(unit, chunk, expert, row0, rows, tile_last);
      int source[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int r = (lt >> 3) + 8 * j;
        // rows past the tile's end repeat its last row (a tile has at least one row)
        const int token = g.sorted_rows[min(row0 + r, tile_last)] >> 3;
        source[j] = token * g.lda + piece * 8;
      }
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag)) { alive = false; timeout(); break; }
        const uint32_t base = smem_base + stage * kStage2Bytes;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int r = (lt >> 3) + 8 * j;
          cp_async_16(base + r * 128 + ((piece ^ (r & 7)) << 4), g.gather_src + source[j] + kb * kBK);
        }
        cp_async_arrive_noinc(leader ? full_bar(stage) : gdone_bar(stage));
        if (++stage == kStages2) { stage = 0; phase ^= 1u; }
      }
    }
    cp_async_wait_all();
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ------------------------------ MMA issuer (leader) ------------------------
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool alive = true;
      for (int unit = pair; unit < total_units && alive; unit += n_pairs, ++local) {
        const int buf = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        if (!mbar_wait_bounded(tempty_bar(buf), (use & 1u) ^ 1u, abort_flag)) { alive = false; timeout(); break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kBN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_bounded(full_bar(stage), phase, abort_flag)) { alive = false; timeout(); break; }
          if (kGather) fence_async_proxy();
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * kStage2Bytes;
          const uint32_t b_addr = a_addr + kStage2ABytes;
          const uint64_t adesc = smem_desc_k_major_sw128(a_addr);
          const uint64_t bdesc = smem_desc_k_major_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            umma_bf16_pair(tmem_d, adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2),
                           kInstrDesc2, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
        if (alive) umma_commit_pair(tfull_bar(buf));
      }
    } else if (lane == 0 && kGather) {
      // ------------------------------ forwarder (peer) ---------------------------
      // this block's gathered rows of a stage have landed: make them visible to the tensor cores and
      // tell the leader, whose MMA reads them
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int unit = pair; unit < total_units && alive; unit += n_pairs) {
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait_bounded(gdone_bar(stage), phase, abort_flag)) { alive = false; timeout(); break; }
          fence_async_proxy();
          mbar_arrive_cluster(map_to_rank(full_bar(stage), 0));
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue (both blocks) ---------------------
    const int ew = (warp - 4) & 3;
    const int eh = (warp - 4) >> 2;
    int local = 0;
    bool alive = true;
    for (int unit = pair; unit < total_units && alive; unit += n_pairs, ++local) {
      int chunk, expert, row0, rows, tile_last;
      unit_tile(unit, chunk, expert, row0, rows, tile_last);
      const int buf = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      if (!mbar_wait_bounded(tfull_bar(buf), use & 1u, abort_flag)) { alive = false; if (lane == 0) timeout(); break; }
      tc_fence_after();
      if (rows > 0)
        drain_accumulator<MODE>(g, pb, tmem_base, buf, ew, eh, lane, store_stage + (warp - 4) * kStoreStageBytes,
                                chunk, row0, rows);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(tempty_bar(buf), 0));
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // neither block leaves while the other may still signal it or read its memory
  if (warp == 2) tmem_dealloc_pair(tmem_base, kTmemColumns);
}

// ---- host side --------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* pointer = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pointer, cudaEnableDefault, &query) == cudaSuccess &&
        query == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(pointer);
    }
  }
  return fn;
}

// 2-D BF16 tensor [rows, cols] row-major, box 64 columns x box_rows rows (128 for tile loads,
// 1 for gather4 loads), 128-byte swizzle.  A descriptor depends only on the base address and these
// numbers, and a layer's weights and the workspace keep their addresses from bind to release, so the
// encoded descriptors are kept: a prefill layer asks for 18 of them per call, always the same ones.
struct MapKey {
  const void* base;
  uint64_t rows, cols, pitch;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.base) * 0x9e3779b97f4a7c15ull;
    h ^= (k.rows + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2));
    h ^= (k.cols * 31 + k.pitch * 131 + k.box_rows + (h << 6) + (h >> 2));
    return static_cast<size_t>(h);
  }
};

bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
              uint32_t box_rows = kBM) {
  static std::mutex mutex;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, cols, pitch_elems, box_rows};
  {
    std::lock_guard<std::mutex> lock(mutex);
    const auto hit = cache.find(key);
    if (hit != cache.end()) { *map = hit->second; return true; }
  }
  PFN_cuTensorMapEncodeTiled_v12000 encode = encode_fn();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_elems * 2};
  const cuuint32_t box[2] = {kBK, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  std::lock_guard<std::mutex> lock(mutex);
  if (cache.size() >= 8192) cache.clear();      // a host that keeps binding new tensors: start over rather than grow
  cache.emplace(key, *map);
  return true;
}

template <int MODE, bool kGather = false>
cudaError_t launch_mode(const TcMaps& maps, const TcProblem& pb, int grid, cudaStream_t stream) {
  const cudaError_t e = opt_in_dynamic_smem<grouped_gemm_tc_kernel<MODE, kGather>>(kTcSmemBytes);
  if (e != cudaSuccess) return e;
  return launch_pdl(grouped_gemm_tc_kernel<MODE, kGather>, dim3(grid), dim3(kTcThreads), kTcSmemBytes, stream, maps, pb);
}

// two-SM form: clusters of two blocks, launched like launch_pdl
template <int MODE, bool kGather>
cudaError_t launch_pair_mode(const TcMaps& maps, const TcProblem& pb, int grid, cudaStream_t stream) {
  const cudaError_t e = opt_in_dynamic_smem<grouped_gemm_tc2_kernel<MODE, kGather>>(kTc2SmemBytes);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid & ~1);
  config.blockDim = dim3(kTcThreads);
  config.dynamicSmemBytes = kTc2SmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 2;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = t_pdl_relaxed ? 1 : 0;
  config.attrs = attributes;
  config.numAttrs = 2;
  return cudaLaunchKernelEx(&config, grouped_gemm_tc2_kernel<MODE, kGather>, maps, pb);
}

}  // namespace

cudaError_t launch_grouped_gemm_tc(GemmMode mode, const GroupedGemm& g, const TcExtra& extra,
                                   cudaStream_t stream) {
  if (g.max_tiles <= 0) return cudaSuccess;
  if (g.k % kBK != 0 || extra.status == nullptr) return cudaErrorInvalidValue;
  TcMaps maps;
  TcProblem pb{};
  pb.g = g;
  pb.status = extra.status;
  pb.n_valid = g.n;
  const bool dual = (mode == kGemmExpertGateUp || mode == kGemmSharedGateUp);
  const uint64_t experts = static_cast<uint64_t>(extra.experts_in_b);
  const bool gather = (mode == kGemmExpertGateUp && g.gather_src != nullptr);
  if (gather && g.sorted_rows == nullptr) return cudaErrorInvalidValue;
  bool ok = make_map(&maps.a, gather ? g.gather_src : g.a, extra.a_rows, static_cast<uint64_t>(g.k),
                     static_cast<uint64_t>(g.lda), gather ? 1u : static_cast<uint32_t>(kBM));
  pb.a_rows = static_cast<int>(extra.a_rows);
  if (mode == kGemmExpertGateUp) {
    pb.n_chunks = g.n / (kBN / 2);
    pb.b_rows_per_expert = 2 * g.n;
    pb.up_row_offset = g.n;
    ok = ok && make_map(&maps.b0, g.b0, experts * 2 * g.n, g.k, g.k);
    maps.b1 = maps.b0;
  } else if (mode == kGemmSharedGateUp) {
    pb.n_chunks = g.n / (kBN / 2);
    pb.b_rows_per_expert = 0;
    pb.up_row_offset = 0;
    ok = ok && make_map(&maps.b0, g.b0, g.n, g.k, g.k) && make_map(&maps.b1, g.b1, g.n, g.k, g.k);
  } else {
    pb.n_chunks = (g.n + kBN - 1) / kBN;
    pb.b_rows_per_expert = (mode == kGemmExpertDown) ? g.n : 0;
    pb.up_row_offset = 0;
    ok = ok && make_map(&maps.b0, g.b0, (mode == kGemmExpertDown ? experts : 1) * static_cast<uint64_t>(g.n), g.k, g.k);
    maps.b1 = maps.b0;
  }
  (void)dual;
  if (!ok) return cudaErrorNotSupported;
  const int grid = extra.sm_count;
  if (extra.pair && g.tile_expert != nullptr && g.parts <= 1) {
    if (mode == kGemmExpertGateUp)
      return gather ? launch_pair_mode<kGemmExpertGateUp, true>(maps, pb, grid, stream)
                    : launch_pair_mode<kGemmExpertGateUp, false>(maps, pb, grid, stream);
    if (mode == kGemmExpertDown) return launch_pair_mode<kGemmExpertDown, false>(maps, pb, grid, stream);
    return cudaErrorInvalidValue;      // the plan holds 256-row tiles: only the two-SM kernels can take them
  }
  switch (mode) {
    case kGemmExpertGateUp:
      return gather ? launch_mode<kGemmExpertGateUp, true>(maps, pb, grid, stream)
                    : launch_mode<kGemmExpertGateUp>(maps, pb, grid, stream);
    case kGemmSharedGateUp: return launch_mode<kGemmSharedGateUp>(maps, pb, grid, stream);
    case kGemmExpertDown: return launch_mode<kGemmExpertDown>(maps, pb, grid, stream);
    case kGemmSharedDown: return launch_mode<kGemmSharedDown>(maps, pb, grid, stream);
    case kGemmPlain: return launch_mode<kGemmPlain>(maps, pb, grid, stream);
    case kGemmPlainF32: return launch_mode<kGemmPlainF32>(maps, pb, grid, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace aima
