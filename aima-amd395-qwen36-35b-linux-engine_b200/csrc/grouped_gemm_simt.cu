// CUDA-core grouped GEMM.  Slow by design (FP32 FMA, 64 x 64 tiles); it exists
// so that the tensor-core kernel can be cross-checked on the device at sizes
// the CPU checker cannot reach.
#include "grouped_gemm.cuh"

namespace aima {
namespace {

constexpr int kBM = 64, kBN = 64, kBK = 32;

template <int MODE>
__global__ void __launch_bounds__(256)
grouped_gemm_simt_kernel(const GroupedGemm g) {
  constexpr bool kDual = (MODE == kGemmExpertGateUp || MODE == kGemmSharedGateUp);
  __shared__ float As[kBK][kBM + 1];
  __shared__ float Bs[kBK][kBN + 1];
  __shared__ float Bs2[kDual ? kBK : 1][kBN + 1];

  const int tile = blockIdx.x;
  const int n_tiles = g.tile_count != nullptr ? *g.tile_count : g.max_tiles;
  if (tile >= n_tiles) return;
  int expert = 0, row0, rows;
  if (g.tile_expert != nullptr) {
    expert = g.tile_expert[tile] - g.expert_base;
    row0 = g.tile_row0[tile];
    rows = g.tile_rows[tile];
  } else {
    row0 = tile * kTileRowsSimt;
    rows = min(kTileRowsSimt, g.dense_rows - row0);
  }
  const int m_base = blockIdx.z * kBM;
  if (m_base >= rows) return;
  const int n0 = blockIdx.y * kBN;

  const __nv_bfloat16* bg = g.b0 + static_cast<size_t>(expert) * g.b_expert_stride;
  const __nv_bfloat16* bu = nullptr;
  if (MODE == kGemmExpertGateUp) bu = bg + static_cast<size_t>(g.n) * g.k;
  if (MODE == kGemmSharedGateUp) bu = g.b1;

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int load_row = tid >> 2, load_k = (tid & 3) * 8;
  float acc[4][4] = {}, acc2[4][4] = {};

  for (int k0 = 0; k0 < g.k; k0 += kBK) {
    {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m_base + load_row < rows)
        v = *reinterpret_cast<const uint4*>(g.a + static_cast<size_t>(row0 + m_base + load_row) * g.lda + k0 + load_k);
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) As[load_k + j][load_row] = f[j];
      const uint4 w = *reinterpret_cast<const uint4*>(bg + static_cast<size_t>(n0 + load_row) * g.k + k0 + load_k);
      unpack8(w, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) Bs[load_k + j][load_row] = f[j];
      if (kDual) {
        const uint4 w2 = *reinterpret_cast<const uint4*>(bu + static_cast<size_t>(n0 + load_row) * g.k + k0 + load_k);
        unpack8(w2, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) Bs2[load_k + j][load_row] = f[j];
      }
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < kBK; ++kk) {
      float a[4], b[4], b2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
      if (kDual) {
#pragma unroll
        for (int j = 0; j < 4; ++j) b2[j] = Bs2[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (kDual) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m_base + ty * 4 + i;
    if (m >= rows) continue;
    const int row = row0 + m;
    float scale = 1.0f;
    if (MODE == kGemmExpertDown) scale = g.row_scale[g.sorted_rows[row]];
    if (MODE == kGemmSharedDown) scale = g.row_scale[row];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      float out;
      if (MODE == kGemmExpertGateUp) {
        const float gate = round_bf16(acc[i][j]);
        const float up = round_bf16(acc2[i][j]);
        out = __fmul_rn(round_bf16(det_silu(gate)), up);
      } else if (MODE == kGemmSharedGateUp) {
        const float gate = round_bf16(acc[i][j]);
        const float up = round_bf16(acc2[i][j]);
        out = __fmul_rn(det_silu(gate), up);
      } else if (MODE == kGemmExpertDown) {
        out = __fmul_rn(acc[i][j], scale);
      } else if (MODE == kGemmSharedDown) {
        out = __fmul_rn(scale, round_bf16(acc[i][j]));
      } else {
        out = acc[i][j];
      }
      g.c[static_cast<size_t>(row) * g.ldc + n] = __float2bfloat16_rn(out);
    }
  }
}

}  // namespace

cudaError_t launch_grouped_gemm_simt(GemmMode mode, const GroupedGemm& g, cudaStream_t stream) {
  if (g.max_tiles <= 0) return cudaSuccess;
  const dim3 grid(g.max_tiles, g.n / kBN, kTileRowsSimt / kBM);
  switch (mode) {
    case kGemmExpertGateUp: grouped_gemm_simt_kernel<kGemmExpertGateUp><<<grid, 256, 0, stream>>>(g); break;
    case kGemmSharedGateUp: grouped_gemm_simt_kernel<kGemmSharedGateUp><<<grid, 256, 0, stream>>>(g); break;
    case kGemmExpertDown: grouped_gemm_simt_kernel<kGemmExpertDown><<<grid, 256, 0, stream>>>(g); break;
    case kGemmSharedDown: grouped_gemm_simt_kernel<kGemmSharedDown><<<grid, 256, 0, stream>>>(g); break;
    case kGemmPlain: grouped_gemm_simt_kernel<kGemmPlain><<<grid, 256, 0, stream>>>(g); break;
    case kGemmPlainF32: return cudaErrorNotSupported;
  }
  return cudaGetLastError();
}

}  // namespace aima
