// Launch interface of the routed-expert FFN, shared by the C-ABI entry points
// and the device-resident decoder.
#pragma once

#include "gemv.cuh"

namespace gufo {

// The stacked expert tensors of one layer as grouped products: `in` = gate and
// up rows of one expert ([2 * expert_ffn] outputs), `down` = its down rows.
struct ExpertBank {
  int experts = 0;
  int expert_ffn = 0;
  int hidden = 0;
  GemvArgs in;
  GemvArgs down;
};

// Checks the handles and shapes of `bank`; ctx->mu is held.
int BuildExpertBank(gufo_cuda_ctx* ctx, const gufo_cuda_expert_bank& bank, ExpertBank* out);

// Top-k routing of `tokens` rows of router outputs (row width `stride`).
int EnqueueRoute(gufo_cuda_ctx* ctx, const float* logits, int stride, int tokens, int experts, int k,
                 int* chosen, float* weights, float* shared_scale);

// y[p] = down_e(silu(gate_e x_p) * up_e x_p) for the pairs with ids[p] = e >= 0.
int EnqueueExpertFfn(gufo_cuda_ctx* ctx, const ExpertBank& bank, const int* ids, int pairs, const float* x,
                     int x_stride, int pairs_per_input, float* ffn, float* act, float* y);

int EnqueueMoeCombine(gufo_cuda_ctx* ctx, const float* shared, const float* scale, const float* weights,
                      const float* expert_out, int tokens, int k, int hidden, float* out);

// Decoder::MoeFfn behind the router: out[t] = shared[t] * scale[t] + the weighted
// sum of the k chosen experts' FFN of x_t (x_t = x + t * x_stride). Two launches
// where the bank's shapes allow (Q4_K, expert_ffn 256 or 512, k <= 8): the gate /
// up product with its SwiGLU, and the down rows with the weighted sum; otherwise
// EnqueueExpertFfn and EnqueueMoeCombine through `ffn` and `expert_out`.
int EnqueueMoeFfn(gufo_cuda_ctx* ctx, const ExpertBank& bank, const int* ids, const float* weights,
                  const float* scale, int tokens, int k, const float* x, int x_stride, const float* shared,
                  float* ffn, float* act, float* expert_out, float* out);

}  // namespace gufo
