/*
 * aima_moe.h -- C ABI of the B200 (sm_100a) routed mixture-of-experts provider.
 *
 * The library replaces the MoE half of one transformer layer of the reference
 * runtime (router -> top-8 -> dispatch plan -> grouped SwiGLU experts +
 * sigmoid-gated shared expert -> weighted combine -> residual add):
 *
 *   prefill  probe_native_q8192_moe_prefill_layer0_oracle
 *            (native/include/aima/native_moe_prefill.h:91-97,
 *             native/src/native_moe_prefill.hip.cpp:543-905)
 *   decode   the MoE half inside run_native_linear_layer / run_native_full_layer
 *            (native/src/native_linear_layer.hip.cpp:163-187,
 *             native/src/native_full_layer.hip.cpp:180-203)
 *
 * Conventions follow the provider ABI the reference runtime already loads with
 * dlopen / ctypes (benchmarks/shape-lab/native/src/qrt_ck_fmha_q8192_provider.cpp
 * :214-325): plain C symbols, raw device pointers, a `void* stream`, and an int
 * status (0 = success).  Positive statuses are cudaError_t values, negative ones
 * are the AIMA_MOE_ERR_* codes below.  Nothing throws across this boundary.
 *
 * Shapes are those of the Qwen3.6-35B-A3B class model: hidden 2048, 256 routed
 * experts, top-8, expert intermediate 512, shared intermediate 512.  All
 * activations and weights are BF16 (uint16_t bit patterns), accumulation FP32.
 *
 * Ownership: the caller owns inputs, outputs and weights.  The library
 * allocates device memory only inside aima_moe_prepare / aima_moe_bind_layer;
 * every *_launch call is asynchronous on the supplied stream and allocates
 * nothing.  One host thread per handle at a time.
 */
#ifndef AIMA_MOE_H_
#define AIMA_MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AIMA_MOE_HIDDEN 2048
#define AIMA_MOE_EXPERTS 256
#define AIMA_MOE_TOP_K 8
#define AIMA_MOE_EXPERT_INTER 512
#define AIMA_MOE_SHARED_INTER 512
#define AIMA_MOE_MAX_LAYERS 64

enum {
  AIMA_MOE_OK = 0,
  AIMA_MOE_ERR_INVALID_ARGUMENT = -1, /* null pointer, bad size, bad layer     */
  AIMA_MOE_ERR_UNSUPPORTED = -2,      /* shape / device the build cannot serve */
  AIMA_MOE_ERR_NOT_BOUND = -3,        /* layer weights were never bound        */
  AIMA_MOE_ERR_ALIAS = -4,            /* output aliases an input               */
  AIMA_MOE_ERR_TIMEOUT = -5,          /* a bounded device-side wait ran out    */
  AIMA_MOE_ERR_INTERNAL = -6,
  AIMA_MOE_ERR_NO_DEVICE = -7,        /* no CUDA device / not an sm_100 part   */
  AIMA_MOE_ERR_CAPACITY = -8          /* tokens exceed the prepared capacity   */
};

typedef struct aima_moe_handle aima_moe_handle;

/* Replaces the constexpr shape block of native_moe_prefill.hip.cpp:28-34 and
 * the owners built in NativeResidentEngine::load
 * (native/src/native_resident_engine.hip.cpp:395-684). */
typedef struct aima_moe_config {
  uint32_t struct_bytes;     /* sizeof(aima_moe_config), ABI check            */
  uint32_t hidden;           /* must be 2048                                  */
  uint32_t experts;          /* must be 256                                   */
  uint32_t top_k;            /* must be 8                                     */
  uint32_t expert_inter;     /* must be 512                                   */
  uint32_t shared_inter;     /* must be 512                                   */
  uint32_t layers;           /* 1 .. AIMA_MOE_MAX_LAYERS                      */
  uint32_t max_prefill_tokens; /* workspace capacity per prefill call; 0 =
                                  decode only                                 */
  uint32_t world;            /* expert-parallel ranks (1, 2, 4, 8)            */
  uint32_t rank;             /* this process' rank                            */
  float rms_eps;             /* 1e-6 in the reference                         */
  uint32_t flags;            /* AIMA_MOE_FLAG_*                               */
} aima_moe_config;

#define AIMA_MOE_FLAG_NONE 0u
/* Qualification only: run the prefill products on CUDA cores instead of the
 * tcgen05 kernel, to cross-check the tensor-core kernel on the device. */
#define AIMA_MOE_FLAG_SIMT_PRODUCTS 1u
/* Qualification only: compute all 256 router logits per token with the canonical
 * FP32 dot instead of filtering candidates with tensor-core logits first. */
#define AIMA_MOE_FLAG_EXACT_ROUTER 2u
/* Prefill, for A/B timing and qualification: copy the routed activation rows into expert order first
 * (one materialised copy read by tiled TMA loads) instead of letting the gate_up tensor-core kernel
 * gather them by token index itself.  Same bits; the default (fused dispatch) saves the copy kernel
 * and 0.5 GB of traffic per T = 8192 layer. */
#define AIMA_MOE_FLAG_MATERIALIZED_DISPATCH 8u
/* Expert-parallel prefill: split the plan's tiles into 2 (or 4) parts and, with copy kernels on two more
 * streams, put the rows of one part into expert order / store the results of another back to their owners
 * while the products of a third run.  Same bits.  It measured no faster than the default, in which the gate_up
 * kernel gathers its rows and the down kernel's epilogue stores its results to their owners itself. */
#define AIMA_MOE_FLAG_EP_PIPELINE_2 32u
#define AIMA_MOE_FLAG_EP_PIPELINE_4 64u
/* Qualification of the certified prefill router: every 64th token is ALSO routed from all 256 canonical
 * logits; aima_moe_metrics counts the tokens audited and those whose expert ids differed.  (The idea of
 * the reference's certified LM head, native/src/native_lm_head_certificate.hip.cpp:33-39, applied to
 * the router; the reference's own router has no filter to audit.) */
#define AIMA_MOE_FLAG_AUDIT_ROUTER 256u
/* Prefill, for A/B timing and qualification: run the expert products in the two-SM form
 * (tcgen05.mma.cta_group::2, a pair of blocks per 256-row tile, each block staging its 128 rows and its half
 * of the weights) instead of the default one-SM form (128-row tiles, one block per tile).  Same bits; on the
 * measured workloads the default is as fast or faster.  Single GPU only. */
#define AIMA_MOE_FLAG_TWO_SM_PRODUCTS 512u
/* Decode, for A/B timing and qualification: do not predict the next layer's experts (its router applied
 * to the current layer's input) and do not request their rows ahead of the routing.  Same bits either
 * way; with the prediction a layer's weight stream overlaps the hand-overs of the previous layer. */
#define AIMA_MOE_FLAG_NO_DECODE_PREDICTION 128u

/* One layer's tensors in checkpoint layout
 * (doc/reference/amd395-qwen36-35b-a3b-bf16/qwen36-shape-manifest.json:162-180,
 * byte sizes enforced as in native_moe_prefill.hip.cpp:588-599 and
 * native/src/native_decode_bindings.hip.cpp:125-135).  With world > 1,
 * expert_gate_up / expert_down hold only this rank's contiguous slab of
 * experts [rank * 256 / world, (rank + 1) * 256 / world). */
typedef struct aima_moe_layer_weights {
  uint32_t struct_bytes;
  uint32_t reserved;
  const void* router;            uint64_t router_bytes;            /* [256,2048]   1 048 576 */
  const void* expert_gate_up;    uint64_t expert_gate_up_bytes;    /* [E_local,1024,2048]    */
  const void* expert_down;       uint64_t expert_down_bytes;       /* [E_local,2048,512]     */
  const void* shared_expert_gate; uint64_t shared_expert_gate_bytes; /* [1,2048]   4 096     */
  const void* shared_gate_proj;  uint64_t shared_gate_proj_bytes;  /* [512,2048]   2 097 152 */
  const void* shared_up_proj;    uint64_t shared_up_proj_bytes;    /* [512,2048]   2 097 152 */
  const void* shared_down_proj;  uint64_t shared_down_proj_bytes;  /* [2048,512]   2 097 152 */
  const void* post_attention_norm; uint64_t post_attention_norm_bytes; /* [2048] 4 096; may be
                                     NULL when only aima_moe_prefill_launch is used */
} aima_moe_layer_weights;

/* Optional per-call views for qualification, the counterpart of the stage
 * buffers compare_native_oracle_tensor reads
 * (native/src/native_moe_prefill.hip.cpp:914-979).  Every member is a device
 * pointer or NULL. */
typedef struct aima_moe_debug_views {
  uint32_t struct_bytes;
  uint32_t reserved;
  void* h2;              /* bf16 [T,2048]  (decode: the norm the kernel formed) */
  void* router_logits;   /* f32  [T,256]   values the selection rule saw; asking for
                            them makes a prefill call use the exact (all-256) router */
  void* topk_ids;        /* i32  [T,8]                                           */
  void* topk_scores;     /* f32  [T,8]                                           */
  void* topk_weights;    /* bf16 [T,8]                                           */
  void* shared_scaled;   /* bf16 [T,2048]                                        */
  void* routed;          /* bf16 [T,2048]                                        */
  void* expert_counts;   /* i32  [256]     prefill only                          */
  void* expert_offsets;  /* i32  [257]     prefill only                          */
  void* sorted_rows;     /* i32  [8T]      prefill only                          */
  void* slot_dots;       /* f32  [8,2048]  decode only: per rank slot, the down
                            product act . Wd before the routing weight           */
  void* slot_rows;       /* bf16 [8T,2048] prefill only (single GPU): weighted expert
                            outputs in (token, slot) order                       */
} aima_moe_debug_views;

/* Counters in the spirit of NativeMoePrefillMetrics
 * (native/include/aima/native_moe_prefill.h:22-35). */
typedef struct aima_moe_metrics {
  uint32_t struct_bytes;
  uint32_t reserved;
  uint64_t prefill_calls;
  uint64_t decode_calls;
  uint64_t kernel_launches;      /* kernels of this library enqueued so far   */
  uint64_t workspace_bytes;      /* device bytes owned by the handle          */
  uint64_t derived_weight_bytes; /* device bytes of re-laid-out weight copies */
  int32_t last_padded_routed_rows; /* block-32 padded rows of the last prefill
                                      call fetched with aima_moe_sync_metrics */
  int32_t device_status;         /* last device status word read              */
  uint64_t router_candidates;    /* experts recomputed exactly by the certified
                                    prefill router since prepare()             */
  uint64_t router_tokens;        /* tokens it routed                           */
  uint64_t router_bound_violations; /* tokens one of whose candidates lay further
                                    from its tensor-core logit than the filter's
                                    bound allows; such a token is routed from all
                                    256 canonical logits instead (expected: 0)  */
  uint64_t router_audited_tokens;   /* AIMA_MOE_FLAG_AUDIT_ROUTER: tokens also
                                    routed from all 256 canonical logits        */
  uint64_t router_audit_mismatches; /* ... whose ids differed (expected: 0)      */
} aima_moe_metrics;

/* Validates the configuration, selects the current CUDA device, allocates the
 * workspace.  Replaces the owner construction in
 * native/src/native_resident_engine.hip.cpp:453-571. */
int aima_moe_prepare(const aima_moe_config* config, aima_moe_handle** handle);

/* Checks and records one layer's weight pointers (name -> tensor resolution of
 * native_moe_prefill.hip.cpp:588-599, native_decode_bindings.hip.cpp:73-106). */
int aima_moe_bind_layer(aima_moe_handle* handle, uint32_t layer,
                        const aima_moe_layer_weights* weights);

/* Harness hook without a counterpart in the reference: an additive FP32 router
 * bias [256] (device pointer, may be NULL) and rounding of router logits to
 * multiples of 1/8, used to build skewed and tie-heavy routing in benchmarks. */
int aima_moe_set_router_hooks(aima_moe_handle* handle, const void* bias_f32,
                              int quantize_eighths);

/* Qualification hook mirroring the reference's "oracle-seeded routing" rerun
 * (native/src/native_moe_prefill.hip.cpp:1059-1123): while set, single-GPU
 * aima_moe_prefill_launch calls of exactly `tokens` rows use these expert ids
 * (int32 [tokens, 8], device) and routing weights (bf16 [tokens, 8], device)
 * instead of the router's, which isolates the expert arithmetic from tie-order
 * effects.  The pointers must stay valid until cleared with (NULL, NULL, 0). */
int aima_moe_set_forced_routing(aima_moe_handle* handle, const int32_t* ids,
                                const void* weights_bf16, uint32_t tokens);

/* Prefill MoE half of `layer` for `tokens` rows.
 * h2 = post-attention RMSNorm output, residual = after_attn, both bf16
 * [tokens,2048]; out bf16 [tokens,2048] = bf16(residual + bf16(routed + shared)).
 * Replaces probe_native_q8192_moe_prefill_layer0_oracle in its production form
 * (collect_oracle_comparisons = false), native_resident_engine.hip.cpp:1061-1094. */
int aima_moe_prefill_launch(aima_moe_handle* handle, uint32_t layer,
                            const void* h2, const void* residual, void* out,
                            uint32_t tokens, const aima_moe_debug_views* debug,
                            void* stream);

/* Decode (one token) MoE half of `layer`: forms h2 = RMSNorm(after_attn) with
 * the bound post-attention norm weight, then router, shared expert, the eight
 * routed experts and the residual add.  after_attn, out: bf16 [2048].
 * Replaces launches[base+4 .. base+9] and the native ops between them in
 * native_linear_layer.hip.cpp:163-187. */
int aima_moe_decode_launch(aima_moe_handle* handle, uint32_t layer,
                           const void* after_attn, void* out,
                           const aima_moe_debug_views* debug, void* stream);

/* Decode through `n_layers` consecutive layers starting at `first_layer` in one
 * persistent launch; layer l+1 consumes layer l's output as its residual
 * stream.  x_in, x_out: bf16 [2048], must not alias. */
int aima_moe_decode_stack_launch(aima_moe_handle* handle, uint32_t first_layer,
                                 uint32_t n_layers, const void* x_in,
                                 void* x_out, void* stream);

/* Prefill through consecutive layers: per layer h2 = RMSNorm(x), residual = x.
 * x_in, x_out: bf16 [tokens,2048]; x_out may equal x_in. */
int aima_moe_prefill_stack_launch(aima_moe_handle* handle, uint32_t first_layer,
                                  uint32_t n_layers, const void* x_in,
                                  void* x_out, uint32_t tokens, void* stream);

/* One prefill layer with the norms on either side of the MoE half fused in, so the host hands
 * over what the attention half produced rather than h2:
 *   after_attn = bf16(attn_out + residual_in); h2 = RMSNorm(after_attn) with the layer's bound
 *   post-attention norm weight     (prefill_add_rmsnorm_2048_kernel, native_pointwise.hip.cpp:144-182;
 *                                   call site four_layer_mini_engine.py:8481-8489)
 *   layer_out = bf16(after_attn + bf16(routed + shared))                    (as aima_moe_prefill_launch)
 *   next_norm_out = RMSNorm(layer_out) with next_norm_weight, written by the combine kernel itself
 *                                   (the next layer's input norm, native_pointwise.hip.cpp:109-142)
 * next_norm_weight / next_norm_out may both be NULL.  All tensors bf16 [tokens,2048]; layer_out
 * may alias residual_in.  World = 1 only. */
int aima_moe_prefill_fused_launch(aima_moe_handle* handle, uint32_t layer, const void* attn_out,
                                  const void* residual_in, const void* next_norm_weight,
                                  void* layer_out, void* next_norm_out, uint32_t tokens, void* stream);

/* Residual add + RMSNorm with the (weight + 1) rule
 * (native/src/native_pointwise.hip.cpp:109-182).  residual may be NULL (plain
 * norm); residual_out may be NULL. */
int aima_moe_rmsnorm_launch(const void* x, const void* residual,
                            const void* weight, void* residual_out,
                            void* norm_out, uint32_t rows, float eps,
                            void* stream);

/* Batch-1 GEMV out[m] = bf16(x[k] . W[m,k]), k in {512, 2048, 4096}: the
 * contract of launch_bf16_wvsplitk (native/src/bf16_wvsplitk.hip.cpp:337-366). */
int aima_moe_gemv_bf16_launch(const void* weight, const void* x, void* out,
                              uint32_t m, uint32_t k, void* stream);

/* Dense D[m,n] = A[m,k] . B[n,k]^T, BF16 in/out, FP32 accumulate on the tensor
 * cores: the contract of Bf16GemmPlan::launch
 * (native/src/bf16_gemm.hip.cpp:220-234).  k % 64 == 0, n % 8 == 0. */
int aima_moe_gemm_bf16_launch(aima_moe_handle* handle, const void* a, const void* b,
                              void* d, uint32_t m, uint32_t n, uint32_t k, void* stream);

/* Decode without any allocation -- this entry point has no counterpart in the
 * reference.  It exists for hosts that must not, or cannot, allocate device
 * memory once they are running: processes that have already given all free HBM
 * to their own weight / KV-cache arenas, and request paths that may not reach
 * cudaMalloc or cudaFree because those calls synchronise the device.  Such hosts
 * cannot use aima_moe_prepare(), which allocates.
 *
 * Runs `n_layers` (1 .. AIMA_MOE_NOALLOC_MAX_LAYERS) consecutive decode layers
 * for one token, exactly like aima_moe_decode_stack_launch: x_in, x_out are
 * bf16 [2048] device vectors that must not alias; `layers[i]` describes layer i
 * with all 256 experts and its post-attention norm weight.  The kernel's scratch
 * lives in one static device array of AIMA_MOE_NOALLOC_SCRATCH_BYTES that every
 * GPU loading the library holds until the process exits; the call itself uses
 * no cudaMalloc / cudaFree or other allocating routine.  If `device_status` is
 * not NULL, the kernel's status word (0 = healthy, see AIMA_MOE_ERR_TIMEOUT) is
 * copied to that device int32 on the stream after the kernel.
 *
 * The first call on each device resolves the address of the static array (the
 * device must be current) and, being the first use of the library's device code
 * there, makes the driver load the module: that is when the driver places the
 * array and the kernel image in device memory.  So make that first call early --
 * before the host hands the remaining HBM to its own arenas, and before starting
 * any stream capture.  Every tensor, x_in, x_out and device_status must be memory
 * of the current device (checked on the host; nothing is enqueued otherwise).
 * Without `device_status` a bounded wait that ran out goes unreported: the next
 * call clears the status word.  All calls on a device share the one array and it keeps the previous
 * call's contents (the call clears the words that must start at zero), so two
 * calls whose kernels overlap on the GPU -- different streams, or different host
 * threads -- race with each other: issue them on one stream or order them with
 * events.  More layers than the maximum are refused with AIMA_MOE_ERR_CAPACITY. */
#define AIMA_MOE_NOALLOC_MAX_LAYERS 8
#define AIMA_MOE_NOALLOC_SCRATCH_BYTES 131072
int aima_moe_decode_layers_noalloc(const aima_moe_layer_weights* layers, uint32_t n_layers,
                                   const void* x_in, void* x_out, float rms_eps,
                                   int32_t* device_status, void* stream);

/* Synchronises the handle's last stream, reads the device status word and the
 * padded-row counter; returns AIMA_MOE_ERR_TIMEOUT if a bounded wait ran out. */
int aima_moe_sync_metrics(aima_moe_handle* handle, aima_moe_metrics* metrics);

/* Expert parallelism over the GPUs of one NVLink / NVSwitch box (no counterpart in
 * the reference, which is single-GPU; it follows from sharding its contiguous
 * per-expert tensors).  A handle prepared with world > 1 binds only its slab of
 * experts and owns one exchange buffer; each rank maps every peer's buffer once:
 *   same process (one host thread per GPU, peer access enabled by the host):
 *       aima_moe_ep_local_buffer on the peer's handle, then
 *       aima_moe_ep_connect(handle, peer, NULL, pointer)
 *   one process per GPU: aima_moe_ep_export -> 64-byte CUDA IPC handle, carried
 *       by the host's own bootstrap (MPI, torch.distributed, a socket), then
 *       aima_moe_ep_connect(handle, peer, ipc_handle, NULL).
 * Decode: every rank evaluates router and shared expert itself, computes the down
 * products of the chosen experts it holds, stores them into the peers' buffers
 * over NVLink and sums all eight in slot order, so every rank ends with the same
 * bits as a single GPU.  All ranks must launch the same layers in the same order.
 * Prefill: tokens are sharded over the ranks (aima_moe_prefill_launch takes this
 * rank's tokens; `max_prefill_tokens` is the GLOBAL capacity, tokens x world must
 * fit).  Each rank stores its activation rows and, once routed, its routing tables
 * into every peer's buffer (all-gathers by peer stores); every rank plans the rows
 * that land on its experts, gathers them from its own copy of the activations
 * inside the gate_up kernel (dispatch), runs its experts, and stores the weighted
 * rows to the owners of their tokens from the down kernel's epilogue (combine).
 * A host that owns a symmetric heap may substitute this rank's own buffer with
 * aima_moe_ep_connect(handle, own rank, NULL, pointer); it must be zero-filled and
 * as large as aima_moe_ep_local_buffer reports. */
int aima_moe_ep_local_buffer(aima_moe_handle* handle, void** pointer, uint64_t* bytes);
int aima_moe_ep_export(aima_moe_handle* handle, void* ipc_handle_64_bytes);
int aima_moe_ep_connect(aima_moe_handle* handle, uint32_t peer, const void* ipc_handle_64_bytes,
                        void* direct_pointer);

/* Tracing, the counterpart of AIMA_NATIVE_PREFILL_TIMELINE
 * (native/src/native_resident_engine.hip.cpp:105-108, 1226-1259): when enabled,
 * the blocks of the decode kernel stamp the GPU's nanosecond timer at
 * AIMA_MOE_DECODE_TRACE_STAMPS points of every layer (layer start, norm done,
 * router/shared rows done, logits arrived, layer plan published, routed gate/up
 * done, activations of all blocks polled and packed, block agrees to go on, first
 * down item landed, down dots done, output stored, down items consumed).  read_decode_timeline synchronises and copies block 0's
 * layers x AIMA_MOE_DECODE_TRACE_STAMPS stamps of the last decode launch. */
#define AIMA_MOE_DECODE_TRACE_STAMPS 12
int aima_moe_set_tracing(aima_moe_handle* handle, int enabled);

/* Qualification only (no counterpart in the reference): sets the device-resident epoch counter from which
 * the decode kernel derives the tags of its exchange words, after synchronising the device.  Tests use it to
 * reach the point where the 16-bit tags of the words between layers come round again (every 65 535 epochs)
 * without running that many layers. */
int aima_moe_debug_set_decode_epoch(aima_moe_handle* handle, uint32_t epoch);
int aima_moe_read_decode_timeline(aima_moe_handle* handle, uint64_t* stamps_ns,
                                  uint32_t capacity, uint32_t* written);
/* The same for EVERY block of the decode kernel, which is what shows the skew between blocks at the
 * kernel's grid-wide hand-overs: *blocks x *layers x AIMA_MOE_DECODE_TRACE_SLOTS words; slots 0-11 as
 * above, 12-15 stamped by the block's copy-issuing warp (router / shared items placed, blind issue
 * over, last gate/up chunk placed, last down item placed).  AIMA_MOE_ERR_CAPACITY if the buffer is
 * too small (at most 256 blocks x AIMA_MOE_MAX_LAYERS). */
#define AIMA_MOE_DECODE_TRACE_SLOTS 16
int aima_moe_read_decode_block_timelines(aima_moe_handle* handle, uint64_t* stamps_ns, uint32_t capacity,
                                         uint32_t* blocks, uint32_t* layers);

/* With tracing on and world > 1: milliseconds of the AIMA_MOE_EP_PREFILL_STAGES
 * stages of the last expert-parallel prefill call on this rank (route, routing
 * exchange, plan, dispatch, expert products, row return, join of the shared expert + wait +
 * combine), from CUDA events on the call's stream. */
#define AIMA_MOE_EP_PREFILL_STAGES 7
int aima_moe_read_ep_prefill_stages(aima_moe_handle* handle, float* stage_ms, uint32_t capacity,
                                    uint32_t* written);

/* Device bytes prepare() would allocate for this configuration. */
int aima_moe_query_workspace(const aima_moe_config* config, uint64_t* bytes);

int aima_moe_release(aima_moe_handle* handle);

/* Message of the last failing call on this thread ("" if none). */
const char* aima_moe_last_error_string(void);

/* ABI version of this header: major << 16 | minor. */
uint32_t aima_moe_abi_version(void);

/* ---------------------------------------------------------------------------
 * LM head with a certified top-1 (the reference's "int8_certified_global_tie" variant).
 * Replaces NativeLmHeadStore::build (native/src/native_lm_head.hip.cpp:126-176: row-wise int8
 * copy, scales and outward-rounded residual norms of lm_head.weight), the row-wise int8 GEMV
 * (benchmarks/shape-lab/four_layer_mini_engine.py:1223-1258, launched at :3570-3590) and
 * launch_native_lm_head_certificate (native/src/native_lm_head_certificate.hip.cpp:213-275,
 * result struct native/include/aima/native_lm_head_certificate.h:21-28).
 *
 * build: weight_bf16 is the raw [rows, 2048] BF16 matrix on the device (248 320 rows in the
 * reference; any row count here).  The library allocates rows x 2048 int8 + 2 x rows floats and
 * quantises on `stream`; the raw matrix stays caller-owned and must outlive the handle (the exact
 * candidate logits are read from it).
 * launch: hidden_bf16 [2048] (the final-norm output), logits_f32 [rows].  Enqueues four kernels:
 * the int8 scan writes approximate logits; rows whose upper bound reaches the largest lower bound
 * become candidates (at most AIMA_MOE_LM_HEAD_CANDIDATES); their exact BF16 logits overwrite the
 * approximate ones in logits_f32; the exact top-1 (equal logits -> lowest token id) goes to the
 * result.  Asynchronous and allocation-free.
 * read_result: synchronises the last stream and copies the result; returns AIMA_MOE_ERR_CAPACITY
 * when more than 1024 rows were candidates (top-1 not certified), as the reference's assert does. */
#define AIMA_MOE_LM_HEAD_CANDIDATES 1024
typedef struct aima_moe_lm_head aima_moe_lm_head;
typedef struct aima_moe_lm_head_result {
  float hidden_l2;             /* ||hidden||_2, rounded up */
  float maximum_lower_bound;   /* largest lower bound over all rows */
  float exact_top1_logit;      /* BF16 value as FP32 */
  uint32_t exact_top1_token_id;
  uint32_t candidate_count;    /* may exceed the capacity; then overflow = 1 */
  uint32_t overflow;
} aima_moe_lm_head_result;

int aima_moe_lm_head_build(const void* weight_bf16, uint32_t rows, aima_moe_lm_head** out, void* stream);
int aima_moe_lm_head_views(aima_moe_lm_head* handle, void** q_weight, void** scales, void** residual_l2);
int aima_moe_lm_head_launch(aima_moe_lm_head* handle, const void* hidden_bf16, void* logits_f32,
                            void* stream);
int aima_moe_lm_head_read_result(aima_moe_lm_head* handle, aima_moe_lm_head_result* result);
int aima_moe_lm_head_release(aima_moe_lm_head* handle);

/* ---------------------------------------------------------------------------
 * Striped weight image: the on-disk format that feeds the expert tensors.  Two lane files
 * (lane0.bin, lane1.bin, meant for two physical drives); every tensor is one extent aligned to 4096
 * bytes in one lane; the aggregate address space is lane 0 followed by lane 1
 * (engine/production-striped-image-manifest.json).
 *
 * image_plan: the reference's layout rule -- sort by descending aligned bytes, then name; give
 *   each tensor to the lane with the smaller total, lane 0 on ties -- reproduces the manifest's
 *   lane / lane_offset / aggregate_offset of all 693 tensors from names and sizes.
 * image_checksum_host: XOR and wrapping SUM over 64-bit words, accumulated into the two outputs
 *   (benchmarks/shape-lab/native/src/striped_image_builder.cpp:137-147).
 * image_build: writes the lane files from host tensors at the planned offsets (zero padding).
 * image_scatter_ingest: the C ABI shape of torch_owned_striped_tensor_scatter_ingest
 *   (benchmarks/shape-lab/native/src/torch_owned_striped_image_loader.hip.cpp:127-135): byte
 *   ranges [aggregate_offsets[i], + payload_bytes[i]) go to the device pointers
 *   destination_ptrs[i]; one reader per lane with two pinned buffers of chunk_bytes and two
 *   streams, O_DIRECT where the file system allows it; then the XOR / SUM checksum of everything
 *   written is evaluated ON THE DEVICE and, if check_expected != 0, compared.  A range need not be
 *   a whole tensor: rank r of W loads the byte range of experts [r*256/W, (r+1)*256/W) of an expert
 *   tensor (offsets stay multiples of 4096).  Synchronous; allocates only its staging buffers. */
typedef struct aima_moe_image_ingest_result {
  uint64_t bytes;         /* payload bytes moved to the device */
  double read_ms;         /* wall time of reads + copies */
  float checksum_ms;      /* device time of the checksum kernel */
  uint32_t direct_io;     /* bit l set: lane l was read with O_DIRECT */
  uint64_t xor_value;
  uint64_t sum_value;
} aima_moe_image_ingest_result;

/* Safetensors shards as the source: safetensors_index lists the tensors of one shard (absolute file
 * offsets: 8 + header length + data_offsets, the manifest's source_offset_bytes); image_build_from_files
 * copies [source_offsets[i], + payload_bytes[i]) of source_paths[i] to the planned extents, as the
 * reference's builder does from its plan rows (striped_image_builder.cpp:97-135).  Pass capacity 0 and
 * entries NULL to count the tensors first. */
typedef struct aima_moe_safetensors_entry {
  char name[200];
  char dtype[8];
  uint32_t rank;
  uint32_t reserved;
  uint64_t shape[4];
  uint64_t data_begin;    /* absolute offset of the first payload byte in the file */
  uint64_t data_end;
} aima_moe_safetensors_entry;
int aima_moe_safetensors_index(const char* path, aima_moe_safetensors_entry* entries, uint64_t capacity,
                               uint64_t* count);
int aima_moe_image_build_from_files(const char* lane0_path, const char* lane1_path,
                                    const char* const* source_paths, const uint64_t* source_offsets,
                                    const uint64_t* payload_bytes, const uint32_t* lane,
                                    const uint64_t* lane_offset, uint64_t count, const uint64_t* lane_bytes,
                                    uint64_t* xor_value, uint64_t* sum_value);
int aima_moe_image_plan(const uint64_t* payload_bytes, const char* const* names, uint64_t count,
                        uint32_t* lane, uint64_t* lane_offset, uint64_t* aggregate_offset,
                        uint64_t* lane_bytes /* [2] */);
int aima_moe_image_checksum_host(const void* data, uint64_t bytes, uint64_t* xor_value, uint64_t* sum_value);
int aima_moe_image_build(const char* lane0_path, const char* lane1_path, const void* const* host_tensors,
                         const uint64_t* payload_bytes, const uint32_t* lane, const uint64_t* lane_offset,
                         uint64_t count, const uint64_t* lane_bytes, uint64_t* xor_value, uint64_t* sum_value);
int aima_moe_image_scatter_ingest(const char* lane0_path, const char* lane1_path,
                                  const uint64_t* aggregate_offsets, const uint64_t* payload_bytes,
                                  const uint64_t* destination_ptrs, uint64_t tensor_count,
                                  uint64_t lane0_bytes, uint64_t lane1_bytes, uint64_t chunk_bytes,
                                  int check_expected, uint64_t expected_xor, uint64_t expected_sum,
                                  aima_moe_image_ingest_result* result);

#ifdef __cplusplus
}
#endif
#endif /* AIMA_MOE_H_ */
