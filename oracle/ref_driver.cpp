// Test infrastructure: launches the reference's own kernels (cut out of the reference checkout into
// ref_extracted.inc by build_ref.py) on the host and exposes them as plain C functions for the
// parity tests.  A launch is a loop over blocks; kernels that synchronise their threads run each
// block's threads as cooperative fibers (ucontext) on the calling thread.  Nothing in the product
// may load the library built from this file.
#include <hip/hip_bf16.h>
#include <hip/hip_bfloat16.h>
#include <hip/hip_runtime.h>

#include <ucontext.h>

#include <cstdio>
#include <cstdlib>
#include <functional>
#include <vector>

ref_dim3 threadIdx, blockIdx, blockDim, gridDim;

namespace {

constexpr std::size_t kFiberStackBytes = 256 * 1024;

struct Fibers {
  ucontext_t main{};
  std::vector<ucontext_t> contexts;
  std::vector<char> stacks;
  std::vector<char> finished;
  const std::function<void()>* body = nullptr;
  int current = -1;
};
Fibers g_fibers;

void fiber_entry() {
  (*g_fibers.body)();
  g_fibers.finished[g_fibers.current] = 1;
  swapcontext(&g_fibers.contexts[g_fibers.current], &g_fibers.main);
}

// Runs body() once per thread of one block.  Each round resumes every unfinished fiber until its next
// __syncthreads() (or its end), so no fiber passes barrier n before all have reached it.
void run_block_with_barriers(unsigned threads, const std::function<void()>& body) {
  Fibers& f = g_fibers;
  f.contexts.resize(threads);
  f.finished.assign(threads, 0);
  f.stacks.resize(static_cast<std::size_t>(threads) * kFiberStackBytes);
  f.body = &body;
  for (unsigned t = 0; t < threads; ++t) {
    getcontext(&f.contexts[t]);
    f.contexts[t].uc_stack.ss_sp = f.stacks.data() + static_cast<std::size_t>(t) * kFiberStackBytes;
    f.contexts[t].uc_stack.ss_size = kFiberStackBytes;
    f.contexts[t].uc_link = &f.main;
    makecontext(&f.contexts[t], fiber_entry, 0);
  }
  unsigned remaining = threads;
  while (remaining != 0) {
    for (unsigned t = 0; t < threads; ++t) {
      if (f.finished[t]) continue;
      f.current = static_cast<int>(t);
      threadIdx.x = t;
      swapcontext(&f.main, &f.contexts[t]);
      if (f.finished[t]) --remaining;
    }
  }
  f.current = -1;
}

template <typename Kernel>
void launch(unsigned grid, unsigned block, bool has_barriers, Kernel kernel) {
  gridDim = ref_dim3{grid, 1, 1};
  blockDim = ref_dim3{block, 1, 1};
  const std::function<void()> body = kernel;
  for (unsigned b = 0; b < grid; ++b) {
    blockIdx = ref_dim3{b, 0, 0};
    if (has_barriers) {
      run_block_with_barriers(block, body);
    } else {
      for (unsigned t = 0; t < block; ++t) {
        threadIdx = ref_dim3{t, 0, 0};
        body();
      }
    }
  }
}

unsigned blocks_for(std::size_t elements, unsigned threads) {
  return static_cast<unsigned>((elements + threads - 1) / threads);
}

}  // namespace

void ref_syncthreads() {
  Fibers& f = g_fibers;
  if (f.current < 0) {
    std::fprintf(stderr, "ref_driver: __syncthreads() outside a fiber launch\n");
    std::abort();
  }
  const int self = f.current;
  swapcontext(&f.contexts[self], &f.main);
  // resumed: the scheduler has restored threadIdx and `current`
}

#include "ref_extracted.inc"

using bf16 = __hip_bfloat16;

extern "C" {

// native_moe_prefill.hip.cpp: launch_router_topk (grid = tokens, 64 threads, thread 0 works)
void ref_router_topk8_softmax(const uint16_t* logits, unsigned tokens, float* scores, int64_t* ids64,
                              int32_t* ids32, uint16_t* weights) {
  launch(tokens, 64, false, [=] {
    ref_moe::router_topk8_softmax_256_kernel(reinterpret_cast<const bf16*>(logits), scores, ids64, ids32,
                                             reinterpret_cast<bf16*>(weights));
  });
}

void ref_shared_silu_multiply(const uint16_t* gate, const uint16_t* up, uint16_t* out, size_t elements) {
  launch(blocks_for(elements, ref_moe::kThreads), ref_moe::kThreads, false, [=] {
    ref_moe::shared_silu_multiply_batched_kernel(reinterpret_cast<const bf16*>(gate), reinterpret_cast<const bf16*>(up),
                                                 reinterpret_cast<bf16*>(out), elements);
  });
}

// gate: one BF16 logit per token; down, out: [tokens, 2048]
void ref_shared_sigmoid_scale(const uint16_t* gate, const uint16_t* down, uint16_t* out, size_t tokens) {
  const size_t elements = tokens * ref_moe::kHidden;
  launch(blocks_for(elements, ref_moe::kThreads), ref_moe::kThreads, false, [=] {
    ref_moe::shared_sigmoid_scale_batched_kernel(reinterpret_cast<const bf16*>(gate), reinterpret_cast<const bf16*>(down),
                                                 reinterpret_cast<bf16*>(out), elements);
  });
}

// gate_up: [rows, 1024] -> activated [rows, 512]
void ref_expert_silu_multiply(const uint16_t* gate_up, uint16_t* activated, size_t rows) {
  const size_t elements = rows * ref_moe::kSharedIntermediate;
  launch(blocks_for(elements, ref_moe::kThreads), ref_moe::kThreads, false, [=] {
    ref_moe::expert_silu_multiply_kernel(reinterpret_cast<const bf16*>(gate_up), reinterpret_cast<bf16*>(activated), elements);
  });
}

// input [tokens, 8, 2048] -> output [tokens, 2048]
void ref_moe_sum8(const uint16_t* input, uint16_t* output, unsigned tokens) {
  launch(tokens, 1024, false, [=] {
    ref_moe::moe_sum8_kernel(reinterpret_cast<const bf16*>(input), reinterpret_cast<bf16*>(output));
  });
}

// topk_ids [routed_rows]; sorted [routed_rows + 256 * 31]; expert_ids [sorted capacity / 32]
void ref_moe_align_block32(const int32_t* topk_ids, size_t routed_rows, int32_t* sorted_token_ids,
                           int32_t* expert_ids, int32_t* num_tokens_post_padded) {
  const size_t capacity = routed_rows + ref_moe::kExperts * (ref_moe::kMoeBlock - 1);
  const size_t blocks = capacity / ref_moe::kMoeBlock;
  launch(1, static_cast<unsigned>(ref_moe::kExperts), true, [=] {
    ref_moe::moe_align_block32_256_kernel(topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded,
                                          routed_rows, capacity, blocks);
  });
}

void ref_bf16_add_pair(const uint16_t* left, const uint16_t* right, const uint16_t* residual,
                       uint16_t* intermediate, uint16_t* output, size_t count) {
  launch(blocks_for(count, ref_pointwise::kThreads), ref_pointwise::kThreads, false, [=] {
    ref_pointwise::bf16_add_pair_kernel(reinterpret_cast<const bf16*>(left), reinterpret_cast<const bf16*>(right),
                                        reinterpret_cast<const bf16*>(residual), reinterpret_cast<bf16*>(intermediate),
                                        reinterpret_cast<bf16*>(output), count);
  });
}

void ref_rmsnorm_2048(const uint16_t* input, const uint16_t* weight, uint16_t* output, unsigned rows) {
  launch(rows, ref_pointwise::kThreads, true, [=] {
    ref_pointwise::prefill_rmsnorm_2048_kernel(reinterpret_cast<const bf16*>(input), reinterpret_cast<const bf16*>(weight),
                                               reinterpret_cast<bf16*>(output));
  });
}

void ref_add_rmsnorm_2048(const uint16_t* input, const uint16_t* residual, const uint16_t* weight,
                          uint16_t* residual_output, uint16_t* norm_output, unsigned rows) {
  launch(rows, ref_pointwise::kThreads, true, [=] {
    ref_pointwise::prefill_add_rmsnorm_2048_kernel(
        reinterpret_cast<const bf16*>(input), reinterpret_cast<const bf16*>(residual), reinterpret_cast<const bf16*>(weight),
        reinterpret_cast<bf16*>(residual_output), reinterpret_cast<bf16*>(norm_output));
  });
}

float ref_rounded_rsqrtf(float value) { return ref_pointwise::pytorch_rounded_rsqrtf(value); }

// decode: shared_input = [gate logit, 512 gate, 512 up] -> activated [512]
void ref_shared_activation(const uint16_t* shared_input, uint16_t* activated) {
  launch(blocks_for(ref_pointwise::kSharedIntermediate, ref_pointwise::kThreads), ref_pointwise::kThreads, false, [=] {
    ref_pointwise::shared_activation_kernel(reinterpret_cast<const bf16*>(shared_input), reinterpret_cast<bf16*>(activated));
  });
}

// decode: out[2048] = bf16(bf16(sigmoid(shared_input[0])) * shared_down)
void ref_shared_gate(const uint16_t* shared_input, const uint16_t* shared_down, uint16_t* output) {
  launch(blocks_for(ref_pointwise::kHidden, ref_pointwise::kThreads), ref_pointwise::kThreads, false, [=] {
    ref_pointwise::shared_gate_kernel(reinterpret_cast<const bf16*>(shared_input), reinterpret_cast<const bf16*>(shared_down),
                                      reinterpret_cast<bf16*>(output));
  });
}

// source [rows, 2048] BF16 -> q [rows, 2048] int8, scales [rows], residual_l2 [rows]
void ref_quantize_lm_head_rows(const uint16_t* source, unsigned rows, int8_t* q_weight, float* scales,
                               float* residual_l2) {
  launch(rows, ref_lm_head::kThreads, true, [=] {
    ref_lm_head::quantize_lm_head_rowwise_kernel(reinterpret_cast<const hip_bfloat16*>(source), q_weight, scales, residual_l2);
  });
}

}  // extern "C"
