/*
 * CPU oracle for the routed mixture-of-experts layer (TEST INFRASTRUCTURE ONLY).
 *
 * This file is a plain-C restatement of the reference engine's MoE half-layer
 * and is used only as the checker in tests, in the smoke check and as the timed
 * CPU baseline of the benchmark.  The product (the CUDA library) never links,
 * loads or calls it.
 *
 * How it is pinned to the reference's own code (the reference repository ships
 * no numeric fixtures for this path; its oracle .bin files are not committed):
 *   - its scalar kernels (top-8 with tie order and softmax, SwiGLU and sigmoid
 *     pointwise stages, 8-way tree sum, add pair, both RMSNorm kernels, block-32
 *     dispatch count, LM-head row quantisation) compiled for the host from the
 *     checkout and run beside every stage (oracle/build_ref.py,
 *     tests/test_oracle_vs_reference_kernels.py);
 *   - its torch functions for the half-layer, cut out of the checkout and
 *     executed (oracle/reference_torch.py, tests/golden/config0_T*.npz);
 *   - its Triton kernels for the batch-1 path, the fused add + RMSNorm and the
 *     LM-head scan, run under Triton's interpreter (oracle/reference_triton.py,
 *     tests/golden/decode_triton_*.npz): ids in order, norm, routing weights,
 *     routed sum and layer output agree bit for bit on the committed cases;
 *   - the order-independent known-answer hashes of its wvSplitK pattern probe
 *     (native/src/bf16_wvsplitk.hip.cpp:218-333,
 *     benchmarks/results/native-wvsplitk-v0.1.0.json:52,73) and the all-ones
 *     GEMM value (native/src/bf16_gemm.hip.cpp:281-291).
 * PARITY UNPINNED for what only the reference's GPU libraries define: the FP32
 * accumulation order of its prefill GEMMs (hipBLASLt, the fused_moe Triton
 * kernel), for which routed-expert values at prefill are held to a tolerance,
 * and the device library's expf beyond one BF16 step.
 *
 * Floating-point contract.  The reference leaves FP32 summation order to its
 * libraries (hipBLASLt, Triton tl.sum).  Routing must be bit-exact, so this
 * oracle fixes ONE order, the same one the CUDA kernels use:
 *
 *   dot(x, w, K)   32 partial sums p[l]; p[l] accumulates, with fused
 *                  multiply-add and in ascending k, every k whose 8-element
 *                  group index (k / 8) is congruent to l modulo 32; the 32
 *                  partials are then combined by the butterfly
 *                  p[l] += p[l ^ s] for s = 16, 8, 4, 2, 1.
 *   sumsq(x)       the order of the reference's RMSNorm kernels
 *                  (native/src/native_pointwise.hip.cpp:109-142): partial t of
 *                  256 adds elements t, t + 256, ... in that order, then the
 *                  partials fold by halving (128, 64, ..., 1).
 *   exp            aima_or_expf below (range reduction + degree-6 polynomial,
 *                  only IEEE fma/mul/add, so CPU and GPU agree bit for bit).
 *   rsqrt          (float)(1.0 / sqrt((double)v)) -- the reference demands the
 *                  correctly rounded FP32 reciprocal square root
 *                  (native/src/native_pointwise.hip.cpp:37-69).
 *
 * Build: gcc -O2 -fPIC -shared -fopenmp -mfma -ffp-contract=off (see Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define AIMA_H 2048      /* hidden size                                        */
#define AIMA_E 256       /* routed experts                                     */
#define AIMA_K 8         /* experts per token                                  */
#define AIMA_I 512       /* expert intermediate size (gate_up rows = 2 * I)    */
#define AIMA_SI 512      /* shared-expert intermediate size                    */

#ifdef __cplusplus
extern "C" {
#endif

/* ----------------------------------------------------------------------- */
/* scalar helpers                                                           */
/* ----------------------------------------------------------------------- */

static inline float bf2f(uint16_t bits) {
  uint32_t u = (uint32_t)bits << 16;
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

/* round-to-nearest-even FP32 -> BF16 (finite inputs; NaN kept quiet) */
static inline uint16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, sizeof u);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

float aima_or_bf16_to_float(uint16_t b) { return bf2f(b); }
uint16_t aima_or_float_to_bf16(float f) { return f2bf(f); }

/* Deterministic e^x.  2^n * P(r), n = rint(x * log2 e), r = x - n ln 2. */
float aima_or_expf(float x) {
  x = fminf(fmaxf(x, -87.0f), 88.0f);
  const float t = x * 1.44269504088896341f;
  const float n = rintf(t);
  float r = fmaf(n, -0.693145751953125f, x);
  r = fmaf(n, -1.42860682030941723e-06f, r);
  float p = 1.0f / 720.0f;
  p = fmaf(p, r, 1.0f / 120.0f);
  p = fmaf(p, r, 1.0f / 24.0f);
  p = fmaf(p, r, 1.0f / 6.0f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  const int32_t e = (int32_t)n + 127;
  const uint32_t scale_bits = (uint32_t)e << 23;
  float scale;
  memcpy(&scale, &scale_bits, sizeof scale);
  return p * scale;
}

static inline float silu_f32(float g) {
  return g / (1.0f + aima_or_expf(-g));
}
static inline float sigmoid_f32(float g) {
  return 1.0f / (1.0f + aima_or_expf(-g));
}

/* canonical dot product, K a multiple of 256 */
float aima_or_dot(const uint16_t* x, const uint16_t* w, int k_size) {
  float p[32];
  for (int l = 0; l < 32; ++l) p[l] = 0.0f;
  for (int i = 0; i < k_size / 256; ++i) {
    for (int l = 0; l < 32; ++l) {
      const int base = 256 * i + 8 * l;
      float acc = p[l];
      for (int j = 0; j < 8; ++j) {
        acc = fmaf(bf2f(x[base + j]), bf2f(w[base + j]), acc);
      }
      p[l] = acc;
    }
  }
  for (int s = 16; s >= 1; s >>= 1) {
    float q[32];
    for (int l = 0; l < 32; ++l) q[l] = p[l] + p[l ^ s];
    memcpy(p, q, sizeof p);
  }
  return p[0];
}

/* Sum of squares of one 2048-wide row in the order of the reference kernels
 * (native/src/native_pointwise.hip.cpp:109-142, prefill_rmsnorm_2048_kernel):
 * thread t of 256 adds the squares of elements t, t+256, ..., t+1792 in that
 * order, then the 256 partials are folded by halving: partial[t] +=
 * partial[t + width] for width = 128, 64, ..., 1.  (The square of a BF16 value
 * is exact in FP32, so a fused and an unfused multiply-add give the same bits.) */
static float sumsq_2048(const uint16_t* x) {
  float part[256];
  for (int t = 0; t < 256; ++t) {
    float acc = 0.0f;
    for (int i = 0; i < 8; ++i) {
      const float v = bf2f(x[t + 256 * i]);
      acc = fmaf(v, v, acc);
    }
    part[t] = acc;
  }
  for (int width = 128; width != 0; width >>= 1)
    for (int t = 0; t < width; ++t) part[t] = part[t] + part[t + width];
  return part[0];
}

static inline float rsqrt_cr(float v) {
  return (float)(1.0 / sqrt((double)v));
}

/* ----------------------------------------------------------------------- */
/* RMSNorm                                                                  */
/* native/src/native_pointwise.hip.cpp:109-182 (prefill_rmsnorm_2048_kernel, */
/* prefill_add_rmsnorm_2048_kernel); four_layer_mini_engine.py:844-885,      */
/* 5127-5128: out = bf16(v * rsqrt(mean(v^2) + eps) * (weight + 1)).         */
/* With `residual` non-null the input is first replaced by bf16(x + residual)*/
/* which is also written to residual_out.                                    */
/* ----------------------------------------------------------------------- */
void aima_or_rmsnorm(const uint16_t* x, const uint16_t* residual,
                     const uint16_t* weight, uint16_t* residual_out,
                     uint16_t* norm_out, int rows, float eps) {
#pragma omp parallel for schedule(static)
  for (int row = 0; row < rows; ++row) {
    uint16_t v[AIMA_H];
    const uint16_t* xr = x + (size_t)row * AIMA_H;
    if (residual != NULL) {
      const uint16_t* rr = residual + (size_t)row * AIMA_H;
      for (int h = 0; h < AIMA_H; ++h) v[h] = f2bf(bf2f(xr[h]) + bf2f(rr[h]));
      if (residual_out != NULL)
        memcpy(residual_out + (size_t)row * AIMA_H, v, sizeof v);
    } else {
      memcpy(v, xr, sizeof v);
    }
    const float inv = rsqrt_cr(sumsq_2048(v) / (float)AIMA_H + eps);
    uint16_t* out = norm_out + (size_t)row * AIMA_H;
    for (int h = 0; h < AIMA_H; ++h) {
      const float scaled = bf2f(v[h]) * inv;
      out[h] = f2bf(scaled * (bf2f(weight[h]) + 1.0f));
    }
  }
}

/* ----------------------------------------------------------------------- */
/* Router                                                                   */
/* ----------------------------------------------------------------------- */

/* FP32 router logits of one token; optional harness-only hooks: an additive
 * per-expert bias and rounding to multiples of 1/8 (the reference has neither;
 * they exist to produce skewed and tie-heavy routing in benchmarks).
 * Prefill: native/src/native_moe_prefill.hip.cpp:829 (router GEMM, FP32
 * accumulate).  Decode: four_layer_mini_engine.py:391-415. */
void aima_or_router_logits(const uint16_t* h2, const uint16_t* router,
                           const float* bias, int quant_eighths,
                           float* logits) {
  for (int e = 0; e < AIMA_E; ++e) {
    float v = aima_or_dot(h2, router + (size_t)e * AIMA_H, AIMA_H);
    if (bias != NULL) v = v + bias[e];
    if (quant_eighths) v = rintf(v * 8.0f) * 0.125f;
    logits[e] = v;
  }
}

static void softmax8(const float* s, float* scores, uint16_t* weights) {
  /* native_moe_prefill.hip.cpp:308-322 and four_layer_mini_engine.py:469-471:
   * exp(s_r - s_0) / sum, s_0 being the largest selected value. */
  float ex[AIMA_K];
  float denom = 0.0f;
  for (int r = 0; r < AIMA_K; ++r) {
    ex[r] = aima_or_expf(s[r] - s[0]);
    denom = denom + ex[r];
  }
  for (int r = 0; r < AIMA_K; ++r) {
    scores[r] = s[r];
    weights[r] = f2bf(ex[r] / denom);
  }
}

/* Prefill selection rule, native/src/native_moe_prefill.hip.cpp:234-323
 * (router_topk8_softmax_256_kernel).  `logits` are the values the rule sees
 * (already BF16-rounded by the caller for the prefill path).
 *   1. threshold = the 8th largest value, counting repeats;
 *   2. take every index whose value exceeds the threshold in ascending index
 *      order, then indices equal to the threshold, ascending, until 8 are held;
 *   3. order the 8 with the fixed bitonic network that exchanges the pair
 *      (left, left ^ stride) when (value[left] > value[right]) equals the
 *      "ascending" flag (left & width) != 0. */
void aima_or_topk_prefill(const float* logits, int32_t* ids, float* scores,
                          uint16_t* weights) {
  int taken[AIMA_K];
  float threshold = 0.0f;
  for (int r = 0; r < AIMA_K; ++r) {
    float best = -INFINITY;
    int best_e = -1;
    for (int e = 0; e < AIMA_E; ++e) {
      int used = 0;
      for (int q = 0; q < r; ++q) used |= (taken[q] == e);
      if (!used && logits[e] > best) {
        best = logits[e];
        best_e = e;
      }
    }
    taken[r] = best_e;
    threshold = best;
  }
  float sv[AIMA_K];
  int si[AIMA_K];
  int n = 0;
  for (int e = 0; e < AIMA_E; ++e)
    if (logits[e] > threshold) { sv[n] = logits[e]; si[n] = e; ++n; }
  for (int e = 0; e < AIMA_E && n < AIMA_K; ++e)
    if (logits[e] == threshold) { sv[n] = logits[e]; si[n] = e; ++n; }
  for (int width = 2; width <= AIMA_K; width *= 2) {
    for (int stride = width / 2; stride > 0; stride /= 2) {
      for (int left = 0; left < AIMA_K; ++left) {
        const int right = left ^ stride;
        if (right <= left) continue;
        const int ascending = (left & width) != 0;
        if ((sv[left] > sv[right]) == ascending) {
          const float tv = sv[left]; sv[left] = sv[right]; sv[right] = tv;
          const int ti = si[left]; si[left] = si[right]; si[right] = ti;
        }
      }
    }
  }
  for (int r = 0; r < AIMA_K; ++r) ids[r] = si[r];
  softmax8(sv, scores, weights);
}

/* Decode selection rule, four_layer_mini_engine.py:416-423, 438-444, 462-468
 * (triton_router_topk_stage1/stage2): eight rounds of arg-max, equal values
 * resolved to the lowest expert id; result in selection order. */
void aima_or_topk_decode(const float* logits, int32_t* ids, float* scores,
                         uint16_t* weights) {
  float v[AIMA_E];
  memcpy(v, logits, sizeof v);
  float sv[AIMA_K];
  for (int r = 0; r < AIMA_K; ++r) {
    float best = -INFINITY;
    int best_e = AIMA_E;
    for (int e = 0; e < AIMA_E; ++e)
      if (v[e] > best) { best = v[e]; best_e = e; }
    if (best_e == AIMA_E) best_e = r; /* all -inf: cannot occur for finite input */
    ids[r] = best_e;
    sv[r] = best;
    v[best_e] = -INFINITY;
  }
  softmax8(sv, scores, weights);
}


/* ----------------------------------------------------------------------- */
/* Pointwise stages, one function per reference kernel so that each can be   */
/* compared with that kernel compiled from the reference checkout.           */
/* ----------------------------------------------------------------------- */

/* shared_silu_multiply_batched_kernel (native_moe_prefill.hip.cpp:210-219) and
 * shared_activation_kernel (native_pointwise.hip.cpp:184-194): SiLU is NOT
 * rounded before the multiply. */
void aima_or_shared_silu_mul(const uint16_t* gate, const uint16_t* up,
                             uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; ++i)
    out[i] = f2bf(silu_f32(bf2f(gate[i])) * bf2f(up[i]));
}

/* shared_sigmoid_scale_batched_kernel (native_moe_prefill.hip.cpp:221-232) and
 * shared_gate_kernel (native_pointwise.hip.cpp:196-205):
 * out = bf16(bf16(sigmoid(gate[token])) * down). */
void aima_or_sigmoid_scale(const uint16_t* gate, const uint16_t* down,
                           uint16_t* out, size_t tokens) {
  for (size_t t = 0; t < tokens; ++t) {
    const float sig = bf2f(f2bf(sigmoid_f32(bf2f(gate[t]))));
    for (int h = 0; h < AIMA_H; ++h)
      out[t * AIMA_H + h] = f2bf(sig * bf2f(down[t * AIMA_H + h]));
  }
}

/* expert_silu_multiply_kernel (native_moe_prefill.hip.cpp:384-402):
 * gate_up [rows, 1024] -> act [rows, 512], SiLU rounded to BF16 first. */
void aima_or_expert_silu_mul(const uint16_t* gate_up, uint16_t* act, size_t rows) {
  for (size_t r = 0; r < rows; ++r)
    for (int i = 0; i < AIMA_I; ++i) {
      const float g = bf2f(gate_up[r * 2 * AIMA_I + i]);
      const float u = bf2f(gate_up[r * 2 * AIMA_I + AIMA_I + i]);
      act[r * AIMA_I + i] = f2bf(bf2f(f2bf(silu_f32(g))) * u);
    }
}

/* moe_sum8_kernel (native_moe_prefill.hip.cpp:404-431): [tokens, 8, 2048] ->
 * [tokens, 2048], FP32 tree (((r0+r4)+(r1+r5))+(r2+r6))+(r3+r7). */
void aima_or_sum8(const uint16_t* in, uint16_t* out, size_t tokens) {
  for (size_t t = 0; t < tokens; ++t) {
    const uint16_t* s = in + t * AIMA_K * AIMA_H;
    for (int h = 0; h < AIMA_H; ++h) {
      const float s04 = bf2f(s[h]) + bf2f(s[4 * AIMA_H + h]);
      const float s15 = bf2f(s[AIMA_H + h]) + bf2f(s[5 * AIMA_H + h]);
      const float s26 = bf2f(s[2 * AIMA_H + h]) + bf2f(s[6 * AIMA_H + h]);
      const float s37 = bf2f(s[3 * AIMA_H + h]) + bf2f(s[7 * AIMA_H + h]);
      float sum = s04 + s15;
      sum = sum + s26;
      sum = sum + s37;
      out[t * AIMA_H + h] = f2bf(sum);
    }
  }
}

/* bf16_add_pair_kernel (native/src/native_pointwise.hip.cpp:94-107). */
void aima_or_add_pair(const uint16_t* left, const uint16_t* right,
                      const uint16_t* residual, uint16_t* intermediate,
                      uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    const uint16_t combined = f2bf(bf2f(left[i]) + bf2f(right[i]));
    if (intermediate) intermediate[i] = combined;
    out[i] = f2bf(bf2f(residual[i]) + bf2f(combined));
  }
}

/* router_topk8_softmax_256_kernel over `tokens` rows of BF16 logits. */
void aima_or_topk_prefill_rows(const uint16_t* logits, int tokens, int32_t* ids,
                               float* scores, uint16_t* weights) {
  for (int t = 0; t < tokens; ++t) {
    float row[AIMA_E];
    for (int e = 0; e < AIMA_E; ++e) row[e] = bf2f(logits[(size_t)t * AIMA_E + e]);
    aima_or_topk_prefill(row, ids + (size_t)t * AIMA_K, scores + (size_t)t * AIMA_K,
                         weights + (size_t)t * AIMA_K);
  }
}

float aima_or_rsqrt(float v) { return rsqrt_cr(v); }

/* ----------------------------------------------------------------------- */
/* Layer weights in checkpoint layout                                       */
/* (doc/reference/amd395-qwen36-35b-a3b-bf16/qwen36-shape-manifest.json:162-180)
 * Expert tensors are passed per expert so that tests may materialise only the
 * experts a case selects; a NULL entry that gets selected is an error.       */
/* ----------------------------------------------------------------------- */
typedef struct {
  const uint16_t* router;            /* [256, 2048]                           */
  const uint16_t* const* gate_up;    /* 256 pointers to [1024, 2048]          */
  const uint16_t* const* down;       /* 256 pointers to [2048, 512]           */
  const uint16_t* shared_gate;       /* [1, 2048]                             */
  const uint16_t* shared_gate_proj;  /* [512, 2048]                           */
  const uint16_t* shared_up_proj;    /* [512, 2048]                           */
  const uint16_t* shared_down_proj;  /* [2048, 512]                           */
  const uint16_t* norm_weight;       /* [2048] post-attention RMSNorm, or NULL*/
  const float* router_bias;          /* [256] or NULL (harness hook)          */
  int32_t router_quant_eighths;      /* harness hook                          */
} aima_or_layer;

typedef struct {
  uint16_t* h2;            /* [T, 2048]   (decode: computed; prefill: echo)   */
  float* logits;           /* [T, 256]    values the selection rule saw       */
  int32_t* ids;            /* [T, 8]                                          */
  float* scores;           /* [T, 8]                                          */
  uint16_t* weights;       /* [T, 8]                                          */
  uint16_t* shared_scaled; /* [T, 2048]                                       */
  uint16_t* routed;        /* [T, 2048]                                       */
} aima_or_debug;

/* shared expert.  prefill: native_moe_prefill.hip.cpp:210-232, 790-826;
 * decode: native/src/native_pointwise.hip.cpp:184-205 + the fused 1025-wide
 * projection (four_layer_mini_engine.py:304-326); torch statement :8286-8303.
 * Both modes round the three projections and the down product to BF16. */
static void shared_expert(const uint16_t* h2, const aima_or_layer* L,
                          uint16_t* shared_scaled) {
  const uint16_t gate_logit = f2bf(aima_or_dot(h2, L->shared_gate, AIMA_H));
  uint16_t gate[AIMA_SI], up[AIMA_SI], act[AIMA_SI], down[AIMA_H];
  for (int i = 0; i < AIMA_SI; ++i) {
    gate[i] = f2bf(aima_or_dot(h2, L->shared_gate_proj + (size_t)i * AIMA_H, AIMA_H));
    up[i] = f2bf(aima_or_dot(h2, L->shared_up_proj + (size_t)i * AIMA_H, AIMA_H));
  }
  aima_or_shared_silu_mul(gate, up, act, AIMA_SI);
  for (int h = 0; h < AIMA_H; ++h)
    down[h] = f2bf(aima_or_dot(act, L->shared_down_proj + (size_t)h * AIMA_SI, AIMA_SI));
  aima_or_sigmoid_scale(&gate_logit, down, shared_scaled, 1);
}

/* Decode MoE half of one layer for ONE token.
 * native/src/native_linear_layer.hip.cpp:163-187 (sequence),
 * four_layer_mini_engine.py:1152-1220 (raw_row_gate_up_activation_kernel,
 * raw_row_down_sum_kernel), native_pointwise.hip.cpp:94-107 (add pair).
 * after_attn [2048] -> out [2048].  Returns 0, or -1 if a selected expert's
 * weights were not supplied. */
int aima_or_decode_layer(const uint16_t* after_attn, const aima_or_layer* L,
                         float eps, uint16_t* out, aima_or_debug* dbg) {
  uint16_t h2[AIMA_H];
  aima_or_rmsnorm(after_attn, NULL, L->norm_weight, NULL, h2, 1, eps);
  float logits[AIMA_E];
  aima_or_router_logits(h2, L->router, L->router_bias,
                        L->router_quant_eighths, logits);
  int32_t ids[AIMA_K];
  float scores[AIMA_K];
  uint16_t weights[AIMA_K];
  aima_or_topk_decode(logits, ids, scores, weights);
  for (int r = 0; r < AIMA_K; ++r)
    if (L->gate_up[ids[r]] == NULL || L->down[ids[r]] == NULL) return -1;

  uint16_t shared_scaled[AIMA_H];
  shared_expert(h2, L, shared_scaled);

  uint16_t act[AIMA_K * AIMA_I];
#pragma omp parallel for schedule(static) collapse(2)
  for (int r = 0; r < AIMA_K; ++r) {
    for (int i = 0; i < AIMA_I; ++i) {
      const uint16_t* wg = L->gate_up[ids[r]] + (size_t)i * AIMA_H;
      const uint16_t* wu = wg + (size_t)AIMA_I * AIMA_H;
      const float g = aima_or_dot(h2, wg, AIMA_H);
      const float u = aima_or_dot(h2, wu, AIMA_H);
      act[r * AIMA_I + i] = f2bf(silu_f32(g) * u);
    }
  }
  uint16_t routed[AIMA_H];
#pragma omp parallel for schedule(static)
  for (int h = 0; h < AIMA_H; ++h) {
    float acc = 0.0f;
    for (int r = 0; r < AIMA_K; ++r) {
      const float d = aima_or_dot(act + r * AIMA_I,
                                  L->down[ids[r]] + (size_t)h * AIMA_I, AIMA_I);
      acc = fmaf(bf2f(weights[r]), d, acc);
    }
    routed[h] = f2bf(acc);
    const float combined = bf2f(f2bf(bf2f(routed[h]) + bf2f(shared_scaled[h])));
    out[h] = f2bf(bf2f(after_attn[h]) + combined);
  }
  if (dbg != NULL) {
    if (dbg->h2) memcpy(dbg->h2, h2, sizeof h2);
    if (dbg->logits) memcpy(dbg->logits, logits, sizeof logits);
    if (dbg->ids) memcpy(dbg->ids, ids, sizeof ids);
    if (dbg->scores) memcpy(dbg->scores, scores, sizeof scores);
    if (dbg->weights) memcpy(dbg->weights, weights, sizeof weights);
    if (dbg->shared_scaled) memcpy(dbg->shared_scaled, shared_scaled, sizeof shared_scaled);
    if (dbg->routed) memcpy(dbg->routed, routed, sizeof routed);
  }
  return 0;
}

/* Prefill MoE half of one layer for the `n_sel` tokens listed in `sel`
 * (NULL = tokens 0..n_sel-1).  native/src/native_moe_prefill.hip.cpp:790-893:
 * BF16-rounded router logits -> prefill selection rule; expert gate_up product
 * rounded to BF16, act = bf16(f32(bf16(silu(g))) * u) (:384-402); down product
 * times the BF16 routing weight rounded to BF16 per slot; slots summed as
 * (((r0+r4)+(r1+r5))+(r2+r6))+(r3+r7) in FP32 (:404-431); then
 * native_pointwise.hip.cpp:94-107.  Outputs are indexed by position in `sel`.
 * h2/residual are the full [T, 2048] inputs. */
int aima_or_prefill_layer(const uint16_t* h2_all, const uint16_t* residual_all,
                          const aima_or_layer* L, const int32_t* sel, int n_sel,
                          uint16_t* out, aima_or_debug* dbg) {
  int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
  for (int s = 0; s < n_sel; ++s) {
    const size_t t = sel ? (size_t)sel[s] : (size_t)s;
    const uint16_t* h2 = h2_all + t * AIMA_H;
    const uint16_t* resid = residual_all + t * AIMA_H;
    float logits[AIMA_E];
    aima_or_router_logits(h2, L->router, L->router_bias,
                          L->router_quant_eighths, logits);
    for (int e = 0; e < AIMA_E; ++e) logits[e] = bf2f(f2bf(logits[e]));
    int32_t ids[AIMA_K];
    float scores[AIMA_K];
    uint16_t weights[AIMA_K];
    aima_or_topk_prefill(logits, ids, scores, weights);
    int missing = 0;
    for (int r = 0; r < AIMA_K; ++r)
      if (L->gate_up[ids[r]] == NULL || L->down[ids[r]] == NULL) missing = 1;
    if (missing) { failed = 1; continue; }

    uint16_t shared_scaled[AIMA_H];
    shared_expert(h2, L, shared_scaled);

    uint16_t* slot_out = (uint16_t*)malloc(sizeof(uint16_t) * AIMA_K * AIMA_H);
    for (int r = 0; r < AIMA_K; ++r) {
      uint16_t gate_up[2 * AIMA_I];
      uint16_t act[AIMA_I];
      for (int i = 0; i < 2 * AIMA_I; ++i)
        gate_up[i] = f2bf(aima_or_dot(h2, L->gate_up[ids[r]] + (size_t)i * AIMA_H, AIMA_H));
      aima_or_expert_silu_mul(gate_up, act, 1);
      const float wr = bf2f(weights[r]);
      for (int h = 0; h < AIMA_H; ++h) {
        const float d = aima_or_dot(act, L->down[ids[r]] + (size_t)h * AIMA_I,
                                    AIMA_I);
        slot_out[r * AIMA_H + h] = f2bf(d * wr);
      }
    }
    uint16_t routed[AIMA_H];
    aima_or_sum8(slot_out, routed, 1);
    aima_or_add_pair(routed, shared_scaled, resid, NULL, out + (size_t)s * AIMA_H, AIMA_H);
    free(slot_out);
    if (dbg != NULL) {
      if (dbg->h2) memcpy(dbg->h2 + (size_t)s * AIMA_H, h2, sizeof(uint16_t) * AIMA_H);
      if (dbg->logits) memcpy(dbg->logits + (size_t)s * AIMA_E, logits, sizeof logits);
      if (dbg->ids) memcpy(dbg->ids + (size_t)s * AIMA_K, ids, sizeof ids);
      if (dbg->scores) memcpy(dbg->scores + (size_t)s * AIMA_K, scores, sizeof scores);
      if (dbg->weights) memcpy(dbg->weights + (size_t)s * AIMA_K, weights, sizeof weights);
      if (dbg->shared_scaled) memcpy(dbg->shared_scaled + (size_t)s * AIMA_H, shared_scaled, sizeof shared_scaled);
      if (dbg->routed) memcpy(dbg->routed + (size_t)s * AIMA_H, routed, sizeof routed);
    }
  }
  return failed ? -1 : 0;
}

/* ----------------------------------------------------------------------- */
/* Dispatch plan                                                            */
/* ----------------------------------------------------------------------- */

/* Deterministic token -> expert plan: per-expert counts, exclusive offsets and
 * the routed rows (flat index token * 8 + slot) grouped by expert, ascending
 * flat index inside an expert (four_layer_mini_engine.py:7806-7823: stable sort
 * of the flattened ids).  Also the reference's block-32 padded row count
 * (native_moe_prefill.hip.cpp:325-382, num_tokens_post_padded). */
void aima_or_dispatch_plan(const int32_t* ids, int tokens, int32_t* counts,
                           int32_t* offsets /* [257] */, int32_t* sorted_rows,
                           int32_t* padded_rows_block32) {
  const int rows = tokens * AIMA_K;
  for (int e = 0; e < AIMA_E; ++e) counts[e] = 0;
  for (int i = 0; i < rows; ++i) counts[ids[i]] += 1;
  offsets[0] = 0;
  int padded = 0;
  for (int e = 0; e < AIMA_E; ++e) {
    offsets[e + 1] = offsets[e] + counts[e];
    padded += (counts[e] + 31) / 32 * 32;
  }
  if (padded_rows_block32) *padded_rows_block32 = padded;
  if (sorted_rows) {
    int32_t cursor[AIMA_E];
    memcpy(cursor, offsets, sizeof cursor);
    for (int i = 0; i < rows; ++i) sorted_rows[cursor[ids[i]]++] = i;
  }
}

/* Batch-1 GEMV out[m] = bf16(dot(x, W[m, :])), the contract of
 * launch_bf16_wvsplitk (native/src/bf16_wvsplitk.hip.cpp:337-366). */
void aima_or_gemv(const uint16_t* weight, const uint16_t* x, uint16_t* out,
                  int m, int k) {
#pragma omp parallel for schedule(static)
  for (int row = 0; row < m; ++row)
    out[row] = f2bf(aima_or_dot(x, weight + (size_t)row * k, k));
}

/* Comparison metrics of compare_native_oracle_tensor
 * (native/src/native_layer_oracle.hip.cpp:136-228) for BF16 tensors:
 * result[0] exact element count, [1] max abs error, [2] relative L2 error,
 * [3] cosine similarity, [4] finite element count. */
void aima_or_compare_bf16(const uint16_t* expected, const uint16_t* actual,
                          size_t n, double* result) {
  double exact = 0, max_abs = 0, se = 0, see = 0, saa = 0, dot = 0, finite = 0;
  for (size_t i = 0; i < n; ++i) {
    const double e = bf2f(expected[i]);
    const double a = bf2f(actual[i]);
    if (expected[i] == actual[i]) exact += 1;
    if (isfinite(a)) finite += 1;
    const double d = a - e;
    if (fabs(d) > max_abs) max_abs = fabs(d);
    se += d * d; see += e * e; saa += a * a; dot += e * a;
  }
  result[0] = exact;
  result[1] = max_abs;
  result[2] = sqrt(se / fmax(see, 1.0e-30));
  result[3] = dot / sqrt(fmax(see * saa, 1.0e-30));
  result[4] = finite;
}


/* ---------------------------------------------------------------------------
 * LM head with a certified top-1.
 * Quantisation: quantize_lm_head_rowwise_kernel (native/src/native_lm_head.hip.cpp:53-115):
 * scale = max(max|w|, 1e-12) * fl(1/127); q = clamp(nearbyint(w / scale), -127, 127);
 * residual_l2 = fl32(sqrt(sum (w - q*scale)^2 in FP64)) moved up 8 ULPs.  The FP64 sum runs as
 * that kernel runs it: 256 partials (columns t, t+256, ...) added pairwise, offset 128 .. 1.
 * Certificate: native/src/native_lm_head_certificate.hip.cpp:44-211.
 * Scan order (this build's statement of the row-wise int8 GEMV, four_layer_mini_engine.py:1223-1258,
 * whose own FP32 order is Triton's): lane l of 32 owns the 16-byte pieces l, l+32, l+64, l+96 of a
 * row, one FP32 fma chain over its 64 weights in ascending order, lanes joined by the butterfly
 * 16, 8, 4, 2, 1; the sum is multiplied by the row's scale.
 * --------------------------------------------------------------------------- */
typedef struct aima_or_lm_head_result {
  float hidden_l2;
  float maximum_lower_bound;
  float exact_top1_logit;
  uint32_t exact_top1_token_id;
  uint32_t candidate_count;
  uint32_t overflow;
} aima_or_lm_head_result;

static double tree256(double* v) {
  for (int offset = 128; offset > 0; offset >>= 1)
    for (int t = 0; t < offset; ++t) v[t] = v[t] + v[t + offset];
  return v[0];
}

void aima_or_lm_head_quantize(const uint16_t* weight, int rows, int8_t* q, float* scales,
                              float* residual_l2) {
#pragma omp parallel for schedule(static)
  for (int row = 0; row < rows; ++row) {
    const uint16_t* w = weight + (size_t)row * 2048;
    float maximum = 0.0f;
    for (int c = 0; c < 2048; ++c) maximum = fmaxf(maximum, fabsf(bf2f(w[c])));
    maximum = fmaxf(maximum, 1.0e-12f);
    const float inverse127 = 1.0f / 127.0f;
    const float scale = maximum * inverse127;
    scales[row] = scale;
    double partial[256];
    for (int t = 0; t < 256; ++t) {
      double local = 0.0;
      for (int c = t; c < 2048; c += 256) {
        const float value = bf2f(w[c]);
        const float rounded = nearbyintf(value / scale);
        const int quantized = (int)fminf(127.0f, fmaxf(-127.0f, rounded));
        q[(size_t)row * 2048 + c] = (int8_t)quantized;
        const float reconstructed = (float)quantized * scale;
        const float residual = value - reconstructed;
        const double product = (double)residual * (double)residual;
        local = local + product;
      }
      partial[t] = local;
    }
    float norm = (float)sqrt(tree256(partial));
    for (int step = 0; step < 8; ++step) norm = nextafterf(norm, INFINITY);
    residual_l2[row] = norm;
  }
}

static float int8_dot_2048(const int8_t* q, const float* x) {
  float lane_acc[32];
  for (int lane = 0; lane < 32; ++lane) {
    float acc = 0.0f;
    for (int piece = 0; piece < 4; ++piece) {
      const int base = 16 * (32 * piece + lane);
      for (int j = 0; j < 16; ++j) acc = fmaf((float)q[base + j], x[base + j], acc);
    }
    lane_acc[lane] = acc;
  }
  for (int offset = 16; offset > 0; offset >>= 1) {
    float next[32];
    for (int lane = 0; lane < 32; ++lane) next[lane] = lane_acc[lane] + lane_acc[lane ^ offset];
    for (int lane = 0; lane < 32; ++lane) lane_acc[lane] = next[lane];
  }
  return lane_acc[0];
}

static int lm_better(float value, uint32_t index, float current, uint32_t current_index) {
  return value > current || (value == current && index < current_index);
}

/* logits [rows]: approximate everywhere, exact (BF16 value) at the candidates.  candidate_ids
 * (capacity 1024) receives the candidates in ascending row order.  Returns 0, or -8 when more
 * than 1024 rows are candidates. */
int aima_or_lm_head_certify(const uint16_t* weight, const int8_t* q, const float* scales,
                            const float* residual_l2, const uint16_t* hidden, int rows,
                            float* logits, aima_or_lm_head_result* result, uint32_t* candidate_ids) {
  float x[2048];
  for (int c = 0; c < 2048; ++c) x[c] = bf2f(hidden[c]);
#pragma omp parallel for schedule(static)
  for (int row = 0; row < rows; ++row)
    logits[row] = int8_dot_2048(q + (size_t)row * 2048, x) * scales[row];
  double partial[256];
  for (int t = 0; t < 256; ++t) {
    double local = 0.0;
    for (int c = t; c < 2048; c += 256) {
      const double value = (double)x[c];
      const double product = value * value;
      local = local + product;
    }
    partial[t] = local;
  }
  float hidden_l2 = (float)sqrt(tree256(partial));
  for (int step = 0; step < 4; ++step) hidden_l2 = nextafterf(hidden_l2, INFINITY);
  float maximum_lower = -INFINITY;
  for (int row = 0; row < rows; ++row) {
    const float error = nextafterf(residual_l2[row] * hidden_l2, INFINITY);
    const float lower = nextafterf(logits[row] - error, -INFINITY);
    maximum_lower = fmaxf(maximum_lower, lower);
  }
  uint32_t count = 0;
  for (int row = 0; row < rows; ++row) {
    const float error = nextafterf(residual_l2[row] * hidden_l2, INFINITY);
    const float upper = nextafterf(logits[row] + error, INFINITY);
    if (upper < maximum_lower) continue;
    if (count < 1024) candidate_ids[count] = (uint32_t)row;
    ++count;
  }
  result->hidden_l2 = hidden_l2;
  result->maximum_lower_bound = maximum_lower;
  result->candidate_count = count;
  result->overflow = count > 1024 ? 1u : 0u;
  const uint32_t bounded = count < 1024 ? count : 1024;
  float best = -INFINITY;
  uint32_t best_index = 0;
  for (uint32_t c = 0; c < bounded; ++c) {
    const uint32_t token = candidate_ids[c];
    const float value = bf2f(f2bf(aima_or_dot(hidden, weight + (size_t)token * 2048, 2048)));
    logits[token] = value;
    if (lm_better(value, token, best, best_index)) { best = value; best_index = token; }
  }
  result->exact_top1_logit = best;
  result->exact_top1_token_id = best_index;
  return count > 1024 ? -8 : 0;
}

#ifdef __cplusplus
}
#endif

/* Prefill routing of `tokens` rows at once (OpenMP over the rows): BF16-rounded logits, then the
 * prefill selection rule; the same two steps aima_or_prefill_layer takes per row. */
void aima_or_router_prefill_rows(const uint16_t* h2, const aima_or_layer* L, int tokens,
                                 float* logits, int32_t* ids, float* scores, uint16_t* weights) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < tokens; ++t) {
    float* row = logits + (size_t)t * AIMA_E;
    aima_or_router_logits(h2 + (size_t)t * AIMA_H, L->router, L->router_bias,
                          L->router_quant_eighths, row);
    for (int e = 0; e < AIMA_E; ++e) row[e] = bf2f(f2bf(row[e]));
    aima_or_topk_prefill(row, ids + (size_t)t * AIMA_K, scores + (size_t)t * AIMA_K,
                         weights + (size_t)t * AIMA_K);
  }
}

/* aima_or_prefill_layer with the routing supplied by the caller for every selected row (ids and BF16
 * weights indexed by position in `sel`): the expert arithmetic alone, as in the reference's
 * "oracle-seeded routing" rerun (native/src/native_moe_prefill.hip.cpp:1059-1123). */
int aima_or_prefill_layer_forced(const uint16_t* h2_all, const uint16_t* residual_all,
                                 const aima_or_layer* L, const int32_t* sel, int n_sel,
                                 const int32_t* forced_ids, const uint16_t* forced_weights,
                                 uint16_t* out, uint16_t* routed_out, uint16_t* shared_out) {
  int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
  for (int s = 0; s < n_sel; ++s) {
    const size_t t = sel ? (size_t)sel[s] : (size_t)s;
    const uint16_t* h2 = h2_all + t * AIMA_H;
    const int32_t* ids = forced_ids + (size_t)s * AIMA_K;
    const uint16_t* weights = forced_weights + (size_t)s * AIMA_K;
    int missing = 0;
    for (int r = 0; r < AIMA_K; ++r)
      if (ids[r] < 0 || ids[r] >= AIMA_E || L->gate_up[ids[r]] == NULL || L->down[ids[r]] == NULL) missing = 1;
    if (missing) { failed = 1; continue; }
    uint16_t shared_scaled[AIMA_H];
    shared_expert(h2, L, shared_scaled);
    uint16_t* slot_out = (uint16_t*)malloc(sizeof(uint16_t) * AIMA_K * AIMA_H);
    for (int r = 0; r < AIMA_K; ++r) {
      uint16_t gate_up[2 * AIMA_I];
      uint16_t act[AIMA_I];
      for (int i = 0; i < 2 * AIMA_I; ++i)
        gate_up[i] = f2bf(aima_or_dot(h2, L->gate_up[ids[r]] + (size_t)i * AIMA_H, AIMA_H));
      aima_or_expert_silu_mul(gate_up, act, 1);
      const float wr = bf2f(weights[r]);
      for (int h = 0; h < AIMA_H; ++h)
        slot_out[r * AIMA_H + h] = f2bf(aima_or_dot(act, L->down[ids[r]] + (size_t)h * AIMA_I, AIMA_I) * wr);
    }
    uint16_t routed[AIMA_H];
    aima_or_sum8(slot_out, routed, 1);
    aima_or_add_pair(routed, shared_scaled, residual_all + t * AIMA_H, NULL, out + (size_t)s * AIMA_H, AIMA_H);
    free(slot_out);
    if (routed_out) memcpy(routed_out + (size_t)s * AIMA_H, routed, sizeof routed);
    if (shared_out) memcpy(shared_out + (size_t)s * AIMA_H, shared_scaled, sizeof shared_scaled);
  }
  return failed ? -1 : 0;
}
