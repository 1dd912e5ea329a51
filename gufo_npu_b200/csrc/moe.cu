// The routed-expert FFN of the MoE models on the device: the router's top-k
// (Route, src/models/qwen35/moe.cpp:16-41 in the reference), the shared
// expert's gate (SharedExpertScale, :43-46), the experts' SwiGLU FFN as grouped
// products over the stacked expert tensors (GgufProjections::ApplyExpert,
// src/models/qwen35/gguf_projections.cpp:218-237) and the weighted sum of
// Decoder::MoeFfn (src/models/qwen35/decoder.cpp:535-557).
//
// The chosen experts stay in device memory from the router kernel to the
// grouped products, so a step never waits for the host. Bytes per token and
// layer: the chosen experts' rows (k * (2 * expert_ffn * hidden + hidden *
// expert_ffn) weights at their GGUF size) plus the router rows; HBM-bound.
#include "moe.cuh"

#include <cfloat>

namespace gufo {

namespace {

constexpr int kRouteThreads = 32;
constexpr int kRouteMaxExperts = 1024;
// The smallest positive normal fp16: the floor of the top-k probability mass
// (moe.cpp:12).
constexpr double kWeightSumFloor = 6.103515625e-5;

// One warp per token; lane l holds experts l, l + 32, ... (PER_LANE of them) in
// registers. Probabilities are exp(logit - max) in double as in the reference;
// their sum is a shuffle tree instead of the reference's index-order loop,
// which can move a weight by the last bit of its fp32 value. The arg-max rounds
// order (probability, id) exactly as the reference does (moe.cpp:28-32).
template <int PER_LANE>
__global__ void __launch_bounds__(kRouteThreads)
RouteKernel(const float* __restrict__ logits, int stride, int experts, int k,
            int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ shared_scale) {
  extern __shared__ double picked[];   // [k]: the chosen probabilities in slot order
  GridDependencyWait();
  const int token = blockIdx.x;
  const float* row = logits + static_cast<size_t>(token) * stride;
  const int lane = threadIdx.x;
  double prob[PER_LANE];
  float top = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    if (e < experts) {
      top = fmaxf(top, row[e]);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    top = fmaxf(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
  }
  const double max_logit = static_cast<double>(top);
  double total = 0;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    // Entries past the end never win a round.
    prob[j] = e < experts ? exp(static_cast<double>(row[e]) - max_logit) : -1.0;
    total += e < experts ? prob[j] : 0.0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    total += __shfl_xor_sync(0xFFFFFFFFu, total, o);
  }
  if (lane == 0 && shared_scale != nullptr) {
    shared_scale[token] = static_cast<float>(1.0 / (1.0 + exp(-static_cast<double>(row[experts]))));
  }
  // k rounds: every lane offers its best remaining entry, the warp keeps the
  // larger probability and the lower id on ties; the winner drops to -1.
  double mass = 0;
  for (int slot = 0; slot < k; ++slot) {
    double best = -2.0;
    int at = 0x7FFFFFFF;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      // Ascending j is ascending id, so a strict compare keeps the lower id.
      if (prob[j] > best) {
        best = prob[j];
        at = lane + 32 * j;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const double other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int other_at = __shfl_xor_sync(0xFFFFFFFFu, at, o);
      if (other > best || (other == best && other_at < at)) {
        best = other;
        at = other_at;
      }
    }
    if ((at & 31) == lane) {
#pragma unroll
      for (int j = 0; j < PER_LANE; ++j) {
        if (j == (at >> 5)) {
          prob[j] = -1.0;
        }
      }
    }
    if (lane == 0) {
      picked[slot] = best;
      chosen[static_cast<size_t>(token) * k + slot] = at;
    }
    // The slot-order sum of the chosen probabilities (moe.cpp:33-36).
    mass += best / total;
  }
  __syncwarp();
  mass = mass > kWeightSumFloor ? mass : kWeightSumFloor;
  for (int slot = lane; slot < k; slot += 32) {
    weights[static_cast<size_t>(token) * k + slot] = static_cast<float>(picked[slot] / total / mass);
  }
}

// out[t][i] = shared[t][i] * scale[t] + sum over slots, in slot order, of
// weights[t][slot] * expert_out[t][slot][i] (decoder.cpp:541-556). `out` may be
// `shared`.
__global__ void __launch_bounds__(256)
CombineKernel(const float* shared, const float* __restrict__ scale,
              const float* __restrict__ weights, const float* __restrict__ expert_out, int k,
              int hidden, float* out) {
  GridDependencyWait();
  const int token = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= hidden) {
    return;
  }
  float v = shared[static_cast<size_t>(token) * hidden + i] * scale[token];
  for (int slot = 0; slot < k; ++slot) {
    v = fmaf(weights[static_cast<size_t>(token) * k + slot],
             expert_out[(static_cast<size_t>(token) * k + slot) * hidden + i], v);
  }
  out[static_cast<size_t>(token) * hidden + i] = v;
}

}  // namespace

int EnqueueRoute(gufo_cuda_ctx* ctx, const float* logits, int stride, int tokens, int experts, int k,
                 int* chosen, float* weights, float* shared_scale) {
  if (tokens <= 0 || experts <= 0 || k <= 0 || k > experts || experts > kRouteMaxExperts || stride < experts) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "route: 1 <= k <= experts <= 1024, stride >= experts");
  }
  const size_t smem = static_cast<size_t>(k) * sizeof(double);
  if (experts <= 256) {
    GUFO_CUDA_TRY(LaunchOverlapped(RouteKernel<8>, dim3(tokens), dim3(kRouteThreads), smem, ctx->stream, 1, logits,
                                   stride, experts, k, chosen, weights, shared_scale));
  } else {
    GUFO_CUDA_TRY(LaunchOverlapped(RouteKernel<32>, dim3(tokens), dim3(kRouteThreads), smem, ctx->stream, 1, logits,
                                   stride, experts, k, chosen, weights, shared_scale));
  }
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

int BuildExpertBank(gufo_cuda_ctx* ctx, const gufo_cuda_expert_bank& bank, ExpertBank* out) {
  if (bank.experts <= 0 || bank.expert_ffn <= 0 || bank.hidden <= 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "expert bank: counts must be positive");
  }
  const struct {
    gufo_cuda_matrix handle;
    int64_t rows, cols;
    const char* name;
  } want[3] = {{bank.gate_exps, bank.expert_ffn, bank.hidden, "ffn_gate_exps"},
               {bank.up_exps, bank.expert_ffn, bank.hidden, "ffn_up_exps"},
               {bank.down_exps, bank.hidden, bank.expert_ffn, "ffn_down_exps"}};
  GemvPart parts[3];
  for (int i = 0; i < 3; ++i) {
    const Matrix* m = ctx->FindMatrix(want[i].handle);
    if (m == nullptr) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, std::string("expert bank: no matrix for ") + want[i].name);
    }
    // Experts are stacked along the rows: [cols, rows, experts] in GGUF terms
    // (gguf_projections.cpp:132-139).
    if (m->cols != want[i].cols || m->rows != want[i].rows * bank.experts) {
      return Fail(GUFO_CUDA_SHAPE, std::string("expert bank: ") + want[i].name + " has shape [" +
                                       std::to_string(m->cols) + ", " + std::to_string(m->rows) +
                                       "], expected [" + std::to_string(want[i].cols) + ", " +
                                       std::to_string(want[i].rows * bank.experts) + "]");
    }
    parts[i] = {m->data, static_cast<int>(want[i].rows), 0, m->type, static_cast<int>(m->row_bytes)};
  }
  out->experts = bank.experts;
  out->expert_ffn = bank.expert_ffn;
  out->hidden = bank.hidden;
  out->in = GemvArgs{};
  out->in.parts[0] = parts[0];
  out->in.parts[1] = parts[1];
  out->in.parts[1].out_offset = bank.expert_ffn;
  out->in.nparts = 2;
  out->in.total_rows = 2 * bank.expert_ffn;
  out->in.y_stride = 2 * bank.expert_ffn;
  out->in.cols = bank.hidden;
  out->down = GemvArgs{};
  out->down.parts[0] = parts[2];
  out->down.nparts = 1;
  out->down.total_rows = bank.hidden;
  out->down.y_stride = bank.hidden;
  out->down.cols = bank.expert_ffn;
  return GUFO_CUDA_OK;
}

int EnqueueExpertFfn(gufo_cuda_ctx* ctx, const ExpertBank& bank, const int* ids, int pairs, const float* x,
                     int x_stride, int pairs_per_input, float* ffn, float* act, float* y) {
  if (pairs <= 0 || ids == nullptr || x == nullptr || ffn == nullptr || y == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "expert ffn: null pointer or no pairs");
  }
  GemvArgs in = bank.in;
  in.x = x;
  in.y = ffn;
  in.group_ids = ids;
  in.groups = pairs;
  in.x_group_stride = x_stride;
  in.x_group_div = pairs_per_input > 1 ? pairs_per_input : 1;
  in.y_group_stride = 2 * bank.expert_ffn;
  GemvArgs down = bank.down;
  down.y = y;
  down.group_ids = ids;
  down.groups = pairs;
  down.y_group_stride = bank.hidden;
  if (act != nullptr && GroupedSwiGluInProduct(ctx, in)) {
    // A block multiplies a gate tile and the up tile of the same rows and stores
    // silu(gate) * up; the down product starts from plain rows.
    in.y = act;
    in.y_group_stride = bank.expert_ffn;
    const int rc = LaunchGemvGrouped(ctx, in, kProloguePlain, nullptr, true);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
    down.x = act;
    down.x_group_stride = bank.expert_ffn;
    return LaunchGemvGrouped(ctx, down, kProloguePlain, nullptr);
  }
  int rc = LaunchGemvGrouped(ctx, in, kProloguePlain, nullptr);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  down.x = ffn;
  down.x_group_stride = 2 * bank.expert_ffn;
  return LaunchGemvGrouped(ctx, down, kPrologueSwiGlu, act);
}

int EnqueueMoeCombine(gufo_cuda_ctx* ctx, const float* shared, const float* scale, const float* weights,
                      const float* expert_out, int tokens, int k, int hidden, float* out) {
  if (tokens <= 0 || k <= 0 || hidden <= 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "moe combine: counts must be positive");
  }
  GUFO_CUDA_TRY(LaunchOverlapped(CombineKernel, dim3((hidden + 255) / 256, tokens), dim3(256), 0, ctx->stream, 1,
                                 shared, scale, weights, expert_out, k, hidden, out));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

}  // namespace gufo

using gufo::Fail;

extern "C" {

int gufo_cuda_route_device(gufo_cuda_ctx* ctx, const float* router, int stride, int tokens, int experts, int k,
                           int* chosen, float* weights, float* shared_scale) {
  if (ctx == nullptr || router == nullptr || chosen == nullptr || weights == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "route: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  if (shared_scale != nullptr && stride < experts + 1) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "route: the shared expert's logit follows the experts'");
  }
  return gufo::EnqueueRoute(ctx, router, stride, tokens, experts, k, chosen, weights, shared_scale);
}

int gufo_cuda_expert_ffn_device(gufo_cuda_ctx* ctx, const gufo_cuda_expert_bank* bank, const int* ids, int pairs,
                                const float* x, int64_t x_stride, int pairs_per_input, float* ffn, float* act,
                                float* y) {
  if (ctx == nullptr || bank == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "expert ffn: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::ExpertBank built;
  const int rc = gufo::BuildExpertBank(ctx, *bank, &built);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  if (x_stride != 0 && x_stride < bank->hidden) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "expert ffn: x_stride is 0 (shared input) or at least hidden");
  }
  if (act == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "expert ffn: null scratch");
  }
  if (pairs_per_input < 1) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "expert ffn: pairs_per_input is at least 1");
  }
  return gufo::EnqueueExpertFfn(ctx, built, ids, pairs, x, static_cast<int>(x_stride), pairs_per_input, ffn, act, y);
}

int gufo_cuda_moe_combine_device(gufo_cuda_ctx* ctx, const float* shared, const float* scale, const float* weights,
                                 const float* expert_out, int tokens, int k, int hidden, float* out) {
  if (ctx == nullptr || shared == nullptr || scale == nullptr || weights == nullptr || expert_out == nullptr ||
      out == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "moe combine: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  return gufo::EnqueueMoeCombine(ctx, shared, scale, weights, expert_out, tokens, k, hidden, out);
}

}  // extern "C"
