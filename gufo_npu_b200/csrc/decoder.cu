// The decode step with every buffer resident on the device: the call sequence
// of qwen35::Decoder::Step (src/models/qwen35/decoder.cpp:478-528 in the
// reference) over this backend's GEMV and DeltaNet kernels, plus the small
// kernels between them (embedding row, residual + RMSNorm, SwiGLU, gated
// attention over the fp16 cache, src/models/qwen35/decoder.cpp:267-412).
//
// One token costs one 4-byte upload (the token id) and one download (the
// logits). The position lives in device memory so that the whole step can be
// replayed as a CUDA graph: two graphs, because the DeltaNet conv window
// alternates between two buffers from step to step.
//
// A step can also take two tokens, the weights read once for both, the second
// a draft that Resolve keeps or rolls back (qwen35_2b::NpuDecoder::Step and
// Resolve, src/models/qwen35_2b/npu_decoder.hpp:57-68).
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <vector>

#include "decode_device.cuh"
#include "gemv.cuh"
#include "moe.cuh"
#include "peer.cuh"
#include "step_kernel.cuh"

namespace gufo {
namespace {

constexpr int kSmallThreads = kTeamThreads;
constexpr int kStepTokens = 2;      // tokens of a pair step
constexpr int kTokenSlots = 8;      // pinned token staging slots of a decoder

__device__ __forceinline__ float SigmoidF(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float SiluF(float x) { return x * SigmoidF(x); }

__device__ __forceinline__ float BlockSum256(float v, float* scratch) {
  v = WarpSum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    scratch[threadIdx.x >> 5] = v;
  }
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kSmallThreads / 32; ++w) {
    total += scratch[w];
  }
  return total;
}

// The embedding row (body in decode_device.cuh). One thread block.
__global__ void __launch_bounds__(kSmallThreads)
EmbedKernel(const __grid_constant__ EmbedArgs a) {
  GridLaunchDependents();
  GridDependencyWait();
  EmbedBody(a, threadIdx.x);
}

// h = h_in + delta (delta when given; h may be h_in), then normed = RMS(h) * w (vec::RmsNorm,
// src/core/vec.hpp:57-63; the residual adds of decoder.cpp:504-506,519-521).
// `advance`, when given, is incremented at the end: the sequence position.
__global__ void __launch_bounds__(kSmallThreads)
AddNormKernel(const float* h_in, float* h, const float* __restrict__ delta,
              const float* __restrict__ w, float eps, int n, float* __restrict__ normed,
              int* advance) {
  __shared__ float scratch[kSmallThreads / 32];
  GridLaunchDependents();
  GridDependencyWait();
  float sq = 0.f;
  for (int i = threadIdx.x; i < n; i += kSmallThreads) {
    float v = h_in[i];
    if (delta != nullptr) {
      v += delta[i];
    }
    if (delta != nullptr || h != h_in) {
      h[i] = v;
    }
    sq = fmaf(v, v, sq);
  }
  const float total = BlockSum256(sq, scratch);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(n) + eps);
  for (int i = threadIdx.x; i < n; i += kSmallThreads) {
    normed[i] = h[i] * inv * w[i];
  }
  if (advance != nullptr && threadIdx.x == 0) {
    *advance += 1;
  }
}

// act[i] = silu(gate[i]) * up[i] over [gate | up] (decoder.cpp:511-514).
__global__ void __launch_bounds__(kSmallThreads)
SwiGluKernel(const float* __restrict__ ffn, int f, float* __restrict__ act) {
  GridLaunchDependents();
  GridDependencyWait();
  const int i = blockIdx.x * kSmallThreads + threadIdx.x;
  if (i < f) {
    act[i] = SiluF(ffn[i]) * ffn[f + i];
  }
}

// Decode attention (bodies in decode_device.cuh). Prep: block h < heads is
// query head h, then one block per KV head. Slices: grid = (splits, kv_heads).
// Merge: grid = heads.
__global__ void __launch_bounds__(kSmallThreads)
AttnPrepKernel(const __grid_constant__ AttnArgs a) {
  __shared__ AttnScratch scratch;
  GridLaunchDependents();
  GridDependencyWait();
  AttnPrepBody(a, blockIdx.x, scratch, threadIdx.x, BlockSync());
}

__global__ void __launch_bounds__(kSmallThreads)
AttnSliceKernel(const __grid_constant__ AttnArgs a) {
  __shared__ AttnScratch scratch;
  GridLaunchDependents();
  GridDependencyWait();
  AttnSliceBody(a, blockIdx.x, blockIdx.y, scratch, threadIdx.x, BlockSync());
}

__global__ void __launch_bounds__(kSmallThreads)
AttnMergeKernel(const __grid_constant__ AttnArgs a) {
  GridLaunchDependents();
  GridDependencyWait();
  AttnMergeBody(a, blockIdx.x, threadIdx.x);
}

template <typename T>
int Upload(gufo_cuda_ctx* ctx, const T* host, size_t n, T** dev) {
  GUFO_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(dev), n * sizeof(T)));
  GUFO_CUDA_TRY(cudaMemcpyAsync(*dev, host, n * sizeof(T), cudaMemcpyHostToDevice, ctx->stream));
  return GUFO_CUDA_OK;
}

int EnqueueAttention(gufo_cuda_ctx* ctx, const AttnArgs& a) {
  const dim3 block(kSmallThreads);
  GUFO_CUDA_TRY(LaunchOverlapped(AttnPrepKernel, dim3(a.heads + a.kv_heads), block, 0, ctx->stream, 1, a));
  GUFO_CUDA_TRY(LaunchOverlapped(AttnSliceKernel, dim3(kAttnSplits, a.kv_heads), block, 0, ctx->stream, 1, a));
  GUFO_CUDA_TRY(LaunchOverlapped(AttnMergeKernel, dim3(a.heads), block, 0, ctx->stream, 1, a));
  ctx->launches.fetch_add(3);
  return GUFO_CUDA_OK;
}

}  // namespace
}  // namespace gufo

extern "C" {

int gufo_cuda_embed_device(gufo_cuda_ctx* ctx, gufo_cuda_matrix matrix, const int* device_token, float* h) {
  if (ctx == nullptr || device_token == nullptr || h == nullptr) {
    return gufo::Fail(GUFO_CUDA_BAD_ARGUMENT, "embed: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  const gufo::Matrix* m = ctx->FindMatrix(matrix);
  if (m == nullptr) {
    return gufo::Fail(GUFO_CUDA_BAD_ARGUMENT, "embed: unknown matrix handle");
  }
  if (m->type != GUFO_CUDA_Q4_K && m->type != GUFO_CUDA_Q6_K && m->type != GUFO_CUDA_F32) {
    return gufo::Fail(GUFO_CUDA_UNSUPPORTED_TYPE, "embed: the lookup runs Q4_K, Q6_K and F32 rows");
  }
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::EmbedArgs a{m->data, m->type, static_cast<int>(m->row_bytes), static_cast<int>(m->cols), device_token, h};
  GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::EmbedKernel, dim3(1), dim3(gufo::kSmallThreads), 0, ctx->stream, 1, a));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

int gufo_cuda_add_rms_norm_device(gufo_cuda_ctx* ctx, float* h, const float* delta, const float* weight,
                                  float eps, int n, float* normed, int* advance) {
  if (ctx == nullptr || h == nullptr || weight == nullptr || normed == nullptr || n <= 0) {
    return gufo::Fail(GUFO_CUDA_BAD_ARGUMENT, "add_rms_norm: bad argument");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::AddNormKernel, dim3(1), dim3(gufo::kSmallThreads), 0, ctx->stream, 1,
                                       static_cast<const float*>(h), h, delta, weight, eps, n, normed, advance));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

int gufo_cuda_swiglu_device(gufo_cuda_ctx* ctx, const float* ffn, int f, float* act) {
  if (ctx == nullptr || ffn == nullptr || act == nullptr || f <= 0) {
    return gufo::Fail(GUFO_CUDA_BAD_ARGUMENT, "swiglu: bad argument");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::SwiGluKernel, dim3((f + gufo::kSmallThreads - 1) / gufo::kSmallThreads),
                                       dim3(gufo::kSmallThreads), 0, ctx->stream, 1, ffn, f, act));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

int gufo_cuda_attention_device(gufo_cuda_ctx* ctx, const gufo_cuda_attention_args* p) {
  if (ctx == nullptr || p == nullptr || p->position == nullptr || p->in == nullptr || p->q_norm == nullptr ||
      p->k_norm == nullptr || p->inv_freq == nullptr || p->keys == nullptr || p->values == nullptr ||
      p->queries == nullptr || p->partials == nullptr || p->ctx_out == nullptr) {
    return gufo::Fail(GUFO_CUDA_BAD_ARGUMENT, "attention: null pointer");
  }
  if (p->kv_heads <= 0 || p->heads % p->kv_heads != 0 || p->heads / p->kv_heads > gufo::kMaxGroup ||
      p->head_dim % 32 != 0 || p->head_dim > 32 * gufo::kMaxPerLane || p->rope_dim > p->head_dim ||
      p->rope_dim % 2 != 0) {
    return gufo::Fail(GUFO_CUDA_SHAPE, "attention: unsupported head shape");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::AttnArgs a{p->heads, p->kv_heads, p->head_dim, p->rope_dim, p->max_positions, p->rms_eps, p->position,
                   p->in, p->q_norm, p->k_norm, p->inv_freq, static_cast<__half*>(p->keys),
                   static_cast<__half*>(p->values), p->queries, p->partials, p->ctx_out};
  return gufo::EnqueueAttention(ctx, a);
}

}  // extern "C"

struct gufo_cuda_decoder {
  gufo_cuda_ctx* ctx = nullptr;
  gufo_cuda_decoder_config c{};
  struct Layer {
    bool attention = false;
    gufo::GemvArgs in, out, ffn_in, ffn_down;
    gufo::GemvArgs router;             // MoE: router rows and the shared expert's gate
    gufo::ExpertBank bank;             // MoE: the stacked expert tensors
    gufo::DeltaNetLayer linear;        // small weights (device), DeltaNet layers
    gufo::DeltaNetGateRows gate_rows{};  // F32 alpha / beta rows, computed inside the mixer kernel
    float* attn_norm = nullptr;
    float* post_norm = nullptr;
    float* q_norm = nullptr;
    float* k_norm = nullptr;
    float* conv[2] = {nullptr, nullptr};
    float* conv_saved = nullptr;       // the window after the first token of a pair
    float* ssm = nullptr;
    float* ssm_spec = nullptr;         // the state after the second token of a pair
    __half* keys = nullptr;
    __half* values = nullptr;
  };
  std::vector<Layer> layers;
  gufo::GemvArgs lm_head;
  gufo::Matrix embed;
  float* output_norm = nullptr;
  float* inv_freq = nullptr;
  // Activations.
  float* h[2] = {nullptr, nullptr};   // the residual stream alternates between two buffers
  float *normed = nullptr, *in = nullptr, *mixed = nullptr, *out = nullptr;
  float* mixed_raw = nullptr;   // DeltaNet outputs before the gated norm (the step kernel)
  float *ffn = nullptr, *act = nullptr, *logits = nullptr, *queries = nullptr, *partials = nullptr;
  // MoE scratch: router outputs, the routing, the experts' intermediate rows.
  float *router = nullptr, *route_weights = nullptr, *shared_scale = nullptr;
  float *expert_ffn = nullptr, *expert_act = nullptr, *expert_out = nullptr;
  int* chosen = nullptr;
  int* position_dev = nullptr;
  int* token_dev = nullptr;      // [kStepTokens]
  // Pinned staging for the token ids: a ring of slots, each reused only after
  // the copy that read it has run (its event), so that steps enqueued without
  // a wait in between never see one another's tokens. The last slot carries the
  // position word Resolve uploads.
  int* token_pinned = nullptr;   // [kTokenSlots + 1][kStepTokens]
  cudaEvent_t token_read[gufo::kTokenSlots] = {};
  unsigned token_slot = 0;
  int position = 0;
  int conv_cur = 0;              // which of a layer's conv windows is current
  int pending = 0;               // tokens of the last step that await Resolve (0 or 2)
  const float* final_h = nullptr;   // final residual rows of the last step (before output_norm)
  // Every DeltaNet layer's windows and states sit in one allocation per kind, so
  // that Resolve moves all layers with one copy.
  float* conv_all[3] = {nullptr, nullptr, nullptr};   // windows 0, 1, saved
  float* ssm_all[2] = {nullptr, nullptr};             // states, draft states
  size_t conv_all_bytes = 0, ssm_all_bytes = 0;
  int steps = 0;
  // Per-stage device time (the reference keeps the same kind of split,
  // NpuDecoder::Timeline, src/models/qwen35_2b/npu_decoder.hpp:121-154).
  bool timeline = false;
  std::vector<cudaEvent_t> marks;
  std::vector<int> mark_kind;
  double stage_ms[GUFO_CUDA_TIMELINE_KINDS] = {};
  int timeline_steps = 0;
  // One graph per (tokens - 1, current conv window, with logits); each kind of
  // step runs eagerly twice first (that sizes staging buffers and sets kernel
  // attributes, which a capture cannot).
  // The last index: 0 no logits, 1 logits on the device, 2 logits on the device
  // and mirrored into `host_mirror` by the LM head's own stores.
  cudaGraphExec_t graph[2][2][3] = {};
  int64_t graph_kernels[2][2][3] = {};
  // A pinned, device-visible host buffer the caller reads logits from: the LM
  // head writes its rows there as well (posted writes over PCIe while the
  // kernel runs), so no copy follows the step. Null: logits are copied down.
  float* host_mirror = nullptr;        // device-side address
  const float* host_mirror_for = nullptr;   // the host pointer it belongs to
  bool mirror_ok = false;              // the LM head is one tensor-core launch
  int eager_runs[2][2] = {};
  std::vector<void*> owned;   // every device allocation, for destroy

  // The one-token step as one persistent kernel (step_kernel.cu), where the
  // model allows it: the program of operations in device memory, two variants
  // (with and without the LM head).
  struct StepPlan {
    bool ok = false;
    int grid = 0;
    int region_bytes = 0;
    gufo::StepOp* ops[2] = {nullptr, nullptr};   // [with logits]
    int nops[2] = {0, 0};
    gufo::StepGemv* gemv = nullptr;
    gufo::StepDelta* delta = nullptr;
    gufo::AttnArgs* attn = nullptr;
    unsigned* sync = nullptr;                    // arrivals, departures, error word
    unsigned long long* stamps = nullptr;        // per-operation time stamps of the last launch
    unsigned* error_pinned = nullptr;            // host copy of the error word
    std::vector<int> op_stage[2];                // timeline kind of each operation
    std::vector<int64_t> op_bytes[2];            // weight / state bytes each operation moves
    int last_with = 0;
    const float* final_h = nullptr;              // the final residual row of a step
    std::string why_not;                         // why the model does not run on it
  } plan;

  int in_width(const Layer& l) const { return l.in.total_rows; }
};

namespace gufo {
namespace {

int Alloc(gufo_cuda_decoder* d, size_t bytes, void** out) {
  GUFO_CUDA_TRY(cudaMalloc(out, bytes));
  d->owned.push_back(*out);
  return GUFO_CUDA_OK;
}

int UploadVec(gufo_cuda_decoder* d, const float* host, size_t n, float** dev, const char* name) {
  if (host == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, std::string("decoder_create: missing vector ") + name);
  }
  int rc = Alloc(d, n * 4, reinterpret_cast<void**>(dev));
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  GUFO_CUDA_TRY(cudaMemcpyAsync(*dev, host, n * 4, cudaMemcpyHostToDevice, d->ctx->stream));
  return GUFO_CUDA_OK;
}

// Stacks whole matrices into one product and checks their shape, as
// GgufProjections' CheckShape does (gguf_projections.cpp:27-46).
int Stack(gufo_cuda_ctx* ctx, const gufo_cuda_matrix* handles, const int64_t* want_rows, int n,
          int64_t want_cols, const char* what, GemvArgs* args) {
  gufo_cuda_rows parts[kMaxParts];
  for (int i = 0; i < n; ++i) {
    const Matrix* m = ctx->FindMatrix(handles[i]);
    if (m == nullptr) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, std::string("decoder_create: no matrix for ") + what);
    }
    if (m->rows != want_rows[i] || m->cols != want_cols) {
      return Fail(GUFO_CUDA_SHAPE, std::string("decoder_create: ") + what + " has shape [" +
                                       std::to_string(m->cols) + ", " + std::to_string(m->rows) +
                                       "], expected [" + std::to_string(want_cols) + ", " +
                                       std::to_string(want_rows[i]) + "]");
    }
    parts[i] = {handles[i], 0, m->rows};
  }
  return BuildGemvArgs(ctx, parts, n, args);
}

#define GUFO_STEP_TRY(expr)           \
  do {                                \
    const int gufo_rc_ = (expr);      \
    if (gufo_rc_ != GUFO_CUDA_OK) {   \
      return gufo_rc_;                \
    }                                 \
  } while (0)

// Where a product's input comes from (FastPrologue, common.cuh). With several
// tokens every pointer is the first of `tokens` rows: residual, pending add and
// plain x `cols` floats apart, a SwiGLU input 2 * cols apart.
struct Input {
  int prologue;
  const float* x = nullptr;        // plain: the rows; SwiGLU: [gate | up] rows
  const float* h_in = nullptr;     // residual + norm
  const float* delta = nullptr;
  int delta_parts = 1;             // vectors to add, delta_stride floats apart
  int delta_stride = 0;
  const float* norm_w = nullptr;
  float* h_out = nullptr;
  int* advance = nullptr;
};

// One stage's product for `tokens` rows with its input fused into the GEMV
// kernels where every part allows it; otherwise the input is materialised by the
// small kernels first. `scratch` holds the materialised / normed rows.
// With `activate` set, `stage` is the stacked gate and up rows of an FFN and y
// receives act = silu(gate) * up ([tokens][rows / 2]) instead of the rows
// themselves, from the product's own epilogue (the reference's
// Epilogue::kSwiGlu, src/npu/gemv.hpp:64-68); the caller has asked
// SwiGluInProduct first.
int FusedProduct(gufo_cuda_ctx* ctx, float rms_eps, const GemvArgs& stage, const Input& in, float* scratch,
                 float* y, int tokens, const PeerOut* peer_out = nullptr, const PeerWait* peer_wait = nullptr,
                 bool activate = false) {
  const dim3 block(kSmallThreads);
  if (activate) {
    FastGemvArgs args{};
    args.cols = stage.cols;
    args.y = y;
    args.y_stride = static_cast<int>(stage.total_rows / 2);
    args.tokens = tokens;
    args.prologue = in.prologue;
    args.x = in.x;
    args.h_in = in.h_in;
    args.delta = in.delta;
    args.delta_parts = in.delta_parts;
    args.delta_stride = in.delta_stride;
    args.norm_w = in.norm_w;
    args.eps = rms_eps;
    args.h_out = in.h_out;
    args.normed_out = in.prologue == kPrologueResNorm ? scratch : nullptr;
    args.advance = in.advance;
    args.epilogue = kEpilogueSwiGlu;
    if (peer_wait != nullptr) {
      args.peer_wait = *peer_wait;
    }
    args.row_bytes = stage.parts[0].row_bytes;
    for (int p = 0; p < 2; ++p) {
      args.parts[args.nparts++] = {stage.parts[p].data, stage.parts[p].rows, stage.parts[p].out_offset};
    }
    return stage.parts[0].type == GUFO_CUDA_Q4_K ? LaunchGemvQ4KFast(ctx, args) : LaunchGemvQ6KFast(ctx, args);
  }
  bool fused = !ctx->force_general && stage.nparts <= kFastMaxParts;
  int fast_parts = 0;
  for (int p = 0; p < stage.nparts; ++p) {
    const int type = stage.parts[p].type;
    if (type == GUFO_CUDA_Q4_K) {
      fused = fused && Q4KFastFits(stage.cols, tokens);
      ++fast_parts;
    } else if (type == GUFO_CUDA_Q6_K) {
      fused = fused && Q6KFastFits(stage.cols, tokens);
      ++fast_parts;
    } else if (in.prologue == kPrologueSwiGlu) {
      fused = false;   // other rows would need the activated vector in memory
    }
  }
  const size_t cols = static_cast<size_t>(stage.cols);
  if (peer_out != nullptr || peer_wait != nullptr) {
    // A product that gathers by itself is one launch of the tensor-core kernel.
    bool one_type = true;
    for (int p = 1; p < stage.nparts; ++p) {
      one_type = one_type && stage.parts[p].type == stage.parts[0].type;
    }
    if (!fused || fast_parts != stage.nparts || !one_type) {
      return Fail(GUFO_CUDA_UNSUPPORTED_TYPE,
                  "matmul_gather: the stage must be up to four Q4_K or Q6_K parts of one format that fit the "
                  "tensor-core GEMV");
    }
  }
  if (in.delta_parts > 1 && (!fused || fast_parts != stage.nparts || tokens != 1)) {
    return Fail(GUFO_CUDA_UNSUPPORTED_TYPE,
                "fused product: several vectors are added to the residual only by the tensor-core GEMV (Q4_K or "
                "Q6_K parts that fit it, one token)");
  }
  if (!fused || fast_parts == 0) {
    const float* x = in.x;
    if (in.prologue == kPrologueResNorm) {
      for (int t = 0; t < tokens; ++t) {
        GUFO_CUDA_TRY(LaunchOverlapped(AddNormKernel, dim3(1), block, 0, ctx->stream, 1, in.h_in + t * cols,
                                       in.h_out + t * cols, in.delta != nullptr ? in.delta + t * cols : nullptr,
                                       in.norm_w, rms_eps, stage.cols, scratch + t * cols, in.advance));
      }
      ctx->launches.fetch_add(tokens);
      x = scratch;
    } else if (in.prologue == kPrologueSwiGlu) {
      for (int t = 0; t < tokens; ++t) {
        GUFO_CUDA_TRY(LaunchOverlapped(SwiGluKernel, dim3((stage.cols + kSmallThreads - 1) / kSmallThreads), block, 0,
                                       ctx->stream, 1, in.x + t * 2 * cols, stage.cols, scratch + t * cols));
      }
      ctx->launches.fetch_add(tokens);
      x = scratch;
    }
    GemvArgs args = stage;
    args.x = x;
    args.y = y;
    return LaunchGemv(ctx, args, tokens);
  }
  bool first = true;
  for (int type : {GUFO_CUDA_Q4_K, GUFO_CUDA_Q6_K}) {
    FastGemvArgs args{};
    args.cols = stage.cols;
    args.y = y;
    args.y_stride = stage.y_stride;
    args.tokens = tokens;
    args.prologue = in.prologue;
    args.x = in.x;
    args.h_in = in.h_in;
    args.delta = in.delta;
    args.delta_parts = in.delta_parts;
    args.delta_stride = in.delta_stride;
    args.norm_w = in.norm_w;
    args.eps = rms_eps;
    args.h_out = in.h_out;
    args.normed_out = in.prologue == kPrologueResNorm ? scratch : nullptr;
    for (int p = 0; p < stage.nparts; ++p) {
      const GemvPart& part = stage.parts[p];
      if (part.type != type) {
        continue;
      }
      args.row_bytes = part.row_bytes;
      args.parts[args.nparts++] = {part.data, part.rows, part.out_offset};
    }
    if (args.nparts == 0) {
      continue;
    }
    args.advance = first ? in.advance : nullptr;
    first = false;
    if (peer_out != nullptr) {
      args.peer_out = *peer_out;
    }
    if (peer_wait != nullptr) {
      args.peer_wait = *peer_wait;
    }
    GUFO_STEP_TRY(type == GUFO_CUDA_Q4_K ? LaunchGemvQ4KFast(ctx, args) : LaunchGemvQ6KFast(ctx, args));
  }
  // Rows of other formats (the F32 alpha / beta rows) read the rows block 0 wrote.
  GemvArgs rest = stage;
  rest.nparts = 0;
  rest.total_rows = 0;
  for (int p = 0; p < stage.nparts; ++p) {
    if (stage.parts[p].type != GUFO_CUDA_Q4_K && stage.parts[p].type != GUFO_CUDA_Q6_K) {
      rest.parts[rest.nparts++] = stage.parts[p];
      rest.total_rows += stage.parts[p].rows;
    }
  }
  if (rest.nparts > 0) {
    rest.x = in.prologue == kPrologueResNorm ? scratch : in.x;
    rest.y = y;
    GUFO_STEP_TRY(LaunchGemv(ctx, rest, tokens));
  }
  return GUFO_CUDA_OK;
}

int FusedProduct(gufo_cuda_decoder* d, const GemvArgs& stage, const Input& in, float* scratch, float* y,
                 int tokens, bool activate = false) {
  return FusedProduct(d->ctx, d->c.rms_eps, stage, in, scratch, y, tokens, nullptr, nullptr, activate);
}

// Whether the gate / up product `stage` can leave silu(gate) * up by itself for
// `tokens` rows: two parts of one tensor-core format with equal whole tiles, and
// a resident thread block for every tile pair.
bool SwiGluInProduct(const gufo_cuda_ctx* ctx, const GemvArgs& stage, int tokens) {
  return !ctx->force_general && stage.nparts == 2 && stage.parts[0].rows == stage.parts[1].rows &&
         stage.parts[0].rows % 16 == 0 && stage.parts[0].type == stage.parts[1].type &&
         FastSwiGluPairsFit(ctx, stage.parts[0].type, stage.cols, tokens, static_cast<int>(stage.parts[0].rows / 16));
}

// Records an event that closes a stage of kind `kind` (timeline mode only).
void Mark(gufo_cuda_decoder* d, int kind) {
  if (!d->timeline) {
    return;
  }
  const size_t used = d->mark_kind.size();
  if (used >= d->marks.size()) {
    cudaEvent_t e;
    cudaEventCreate(&e);
    d->marks.push_back(e);
  }
  cudaEventRecord(d->marks[used], d->ctx->stream);
  d->mark_kind.push_back(kind);
}

// `tokens` (1 or 2) rows from the current position in one pass: every product
// runs once for all rows, the mixers token by token (the second sees the
// first's cache row and state). With two tokens the DeltaNet layers leave the
// state after the first token in ssm and the window after it in conv_saved; the
// second token's go to ssm_spec and the other conv window (DeltaNetStep::Run,
// src/models/qwen35_2b/deltanet.hpp:35-44). Token t's rows sit at t * width in
// every activation buffer.
int EnqueueStep(gufo_cuda_decoder* d, int parity, bool want_logits, int tokens, bool mirror = false) {
  gufo_cuda_ctx* ctx = d->ctx;
  const gufo_cuda_decoder_config& c = d->c;
  cudaStream_t st = ctx->stream;
  const dim3 one(1), block(kSmallThreads);
  const size_t hidden = static_cast<size_t>(c.hidden);
  int cur = 0;   // which residual buffer is current
  for (int t = 0; t < tokens; ++t) {
    EmbedArgs embed{d->embed.data, d->embed.type, static_cast<int>(d->embed.row_bytes), c.hidden,
                    d->token_dev + t, d->h[0] + t * hidden};
    GUFO_CUDA_TRY(LaunchOverlapped(EmbedKernel, one, block, 0, st, 1, embed));
  }
  ctx->launches.fetch_add(tokens);
  Mark(d, -1);
  Mark(d, GUFO_CUDA_TIMELINE_EMBED);
  const float* pending = nullptr;   // projection output not yet added to the residual
  for (int il = 0; il < c.layers; ++il) {
    auto& l = d->layers[il];
    Input norm1{kPrologueResNorm};
    norm1.h_in = d->h[cur];
    norm1.delta = pending;
    norm1.norm_w = l.attn_norm;
    norm1.h_out = d->h[cur ^ 1];
    GUFO_STEP_TRY(FusedProduct(d, l.in, norm1, d->normed, d->in, tokens));
    Mark(d, GUFO_CUDA_TIMELINE_IN);
    cur ^= 1;
    const size_t in_width = static_cast<size_t>(l.in.y_stride);
    const size_t mixed_width = static_cast<size_t>(l.out.cols);
    for (int t = 0; t < tokens; ++t) {
      const float* in = d->in + t * in_width;
      float* mixed = d->mixed + t * mixed_width;
      if (l.attention) {
        AttnArgs a{c.heads, c.kv_heads, c.head_dim, c.rope_dim, c.max_positions, c.rms_eps,
                   d->position_dev, in, l.q_norm, l.k_norm, d->inv_freq, l.keys, l.values,
                   d->queries, d->partials, mixed, t};
        GUFO_STEP_TRY(EnqueueAttention(ctx, a));
      } else {
        // One token: window to window, state in place. Two: the first goes to
        // conv_saved, the second from there to the other window and ssm_spec.
        const bool last = t == tokens - 1;
        const float* conv_from = t == 0 ? l.conv[parity] : l.conv_saved;
        float* conv_to = last ? l.conv[parity ^ 1] : l.conv_saved;
        gufo_cuda_linear_seq seq{in, conv_from, conv_to, l.ssm, t > 0 ? l.ssm_spec : nullptr, mixed};
        gufo::DeltaNetGateRows gate_rows = l.gate_rows;
        gate_rows.x = d->normed + t * hidden;
        // A second token reads the state the launch before it wrote: no early loads.
        GUFO_STEP_TRY(EnqueueDeltaNetLinear(ctx, l.linear, &seq, 1, t == 0,
                                            gate_rows.alpha_w != nullptr ? &gate_rows : nullptr));
      }
    }
    Mark(d, l.attention ? GUFO_CUDA_TIMELINE_ATTENTION : GUFO_CUDA_TIMELINE_DELTANET);
    Input plain{kProloguePlain};
    plain.x = d->mixed;
    GUFO_STEP_TRY(FusedProduct(d, l.out, plain, d->act, d->out, tokens));
    Mark(d, GUFO_CUDA_TIMELINE_OUT);
    Input norm2{kPrologueResNorm};
    norm2.h_in = d->h[cur];
    norm2.delta = d->out;
    norm2.norm_w = l.post_norm;
    norm2.h_out = d->h[cur ^ 1];
    // Where it can, the gate / up product leaves silu(gate) * up (its kernel's
    // epilogue) and the down product starts from plain rows; else the
    // activation is the down product's fused input.
    const bool activate = SwiGluInProduct(ctx, l.ffn_in, tokens);
    GUFO_STEP_TRY(FusedProduct(d, l.ffn_in, norm2, d->normed, activate ? d->act : d->ffn, tokens, activate));
    Mark(d, GUFO_CUDA_TIMELINE_FFN_IN);
    cur ^= 1;
    Input down_in{activate ? kProloguePlain : kPrologueSwiGlu};
    down_in.x = activate ? d->act : d->ffn;
    GUFO_STEP_TRY(FusedProduct(d, l.ffn_down, down_in, activate ? d->normed : d->act, d->out, tokens));
    if (c.experts > 0) {
      // Decoder::MoeFfn (decoder.cpp:535-557): d->out holds the shared
      // expert's output, d->normed the layer's normed input.
      GemvArgs router = l.router;
      router.x = d->normed;
      router.y = d->router;
      GUFO_STEP_TRY(LaunchGemv(ctx, router, tokens));
      GUFO_STEP_TRY(EnqueueRoute(ctx, d->router, c.experts + 1, tokens, c.experts, c.experts_used, d->chosen,
                                 d->route_weights, d->shared_scale));
      GUFO_STEP_TRY(EnqueueMoeFfn(ctx, l.bank, d->chosen, d->route_weights, d->shared_scale, tokens, c.experts_used,
                                  d->normed, c.hidden, d->out, d->expert_ffn, d->expert_act, d->expert_out, d->out));
    }
    Mark(d, GUFO_CUDA_TIMELINE_FFN_DOWN);
    pending = d->out;
  }
  Input last{kPrologueResNorm};
  last.h_in = d->h[cur];
  last.delta = pending;
  last.norm_w = d->output_norm;
  last.h_out = d->h[cur ^ 1];
  last.advance = d->position_dev;
  d->final_h = last.h_out;
  if (want_logits && mirror) {
    // The logits go to the device buffer and, by the same stores, to the
    // caller's pinned host buffer.
    PeerOut both{};
    both.world = 2;
    both.rank = 0;
    both.slot = -1;
    both.y[0] = d->logits;
    both.y[1] = d->host_mirror;
    GUFO_STEP_TRY(FusedProduct(ctx, c.rms_eps, d->lm_head, last, d->normed, d->logits, tokens, &both, nullptr));
  } else if (want_logits) {
    GUFO_STEP_TRY(FusedProduct(d, d->lm_head, last, d->normed, d->logits, tokens));
  } else {
    // A prompt pass whose logits nobody reads: only the final residuals.
    for (int t = 0; t < tokens; ++t) {
      GUFO_CUDA_TRY(LaunchOverlapped(AddNormKernel, one, block, 0, st, 1, last.h_in + t * hidden,
                                     last.h_out + t * hidden, last.delta + t * hidden, last.norm_w, c.rms_eps,
                                     c.hidden, d->normed + t * hidden, last.advance));
    }
    ctx->launches.fetch_add(tokens);
  }
  Mark(d, GUFO_CUDA_TIMELINE_LM_HEAD);
  return GUFO_CUDA_OK;
}

// Describes the one-token step of `d` as a program for the persistent kernel.
// Leaves plan.ok false, with the reason, when the model needs something the
// kernel does not do: the launch chain (EnqueueStep) then runs every step.
int BuildStepPlan(gufo_cuda_decoder* d) {
  auto& plan = d->plan;
  gufo_cuda_ctx* ctx = d->ctx;
  const gufo_cuda_decoder_config& c = d->c;
  auto no = [&](const std::string& why) {
    plan.why_not = why;
    return GUFO_CUDA_OK;
  };
  if (c.experts > 0) {
    return no("MoE layers run on the launch chain");
  }
  std::vector<StepGemv> gemv;
  std::vector<StepDelta> delta;
  std::vector<AttnArgs> attn;
  struct HostOp {
    StepOp op;
    int stage;
    int64_t bytes;
  };
  std::vector<HostOp> ops;
  int region = StepScratchBytes();
  int max_split = 1;
  std::string problem;
  // One product of the step. `split`: the consumer adds partial vectors, so a
  // product over more than one slab of K may be cut into (tile, slab) items.
  auto product = [&](const GemvArgs& stage, int rows_limit, bool split, float* y, int stage_kind) -> int {
    StepGemv g{};
    int64_t bytes = 0;
    g.nparts = 0;
    for (int p = 0; p < stage.nparts && rows_limit != 0; ++p) {
      const GemvPart& part = stage.parts[p];
      if (g.nparts == kFastMaxParts) {
        problem = "a stage stacks more than four matrices";
        return -1;
      }
      if (g.nparts == 0) {
        g.type = part.type;
        g.row_bytes = part.row_bytes;
      }
      if ((part.type != GUFO_CUDA_Q4_K && part.type != GUFO_CUDA_Q6_K) || part.type != g.type) {
        problem = "a stage mixes block formats, or has rows that are neither Q4_K nor Q6_K";
        return -1;
      }
      if ((reinterpret_cast<uintptr_t>(part.data) & 15) != 0 || part.row_bytes % 16 != 0) {
        problem = "weight rows are not 16-byte aligned";
        return -1;
      }
      g.parts[g.nparts++] = {part.data, part.rows, part.out_offset};
      g.tiles += (part.rows + 15) / 16;
      bytes += static_cast<int64_t>(part.rows) * RowBytes(part.type, stage.cols);
    }
    if (g.nparts == 0) {
      g.type = GUFO_CUDA_Q4_K;   // a norm without a product (a step without logits)
    }
    g.cols = stage.cols;
    if (g.cols % kSuperBlock != 0) {
      problem = "a product's input is not a whole number of 256-value blocks";
      return -1;
    }
    g.slabs_per_tile = (g.cols / kSuperBlock + 7) / 8;
    g.split = split && g.slabs_per_tile > 1 ? 1 : 0;
    g.y = y;
    g.y_stride = stage.y_stride;
    g.y_split_stride = c.hidden;
    region = std::max(region, StepImageBytes(g.type, g.cols));
    if (g.split) {
      max_split = std::max(max_split, g.slabs_per_tile);
    }
    HostOp h{};
    h.op.kind = kStepGemv;
    h.op.items = g.split ? g.tiles * g.slabs_per_tile : g.tiles;
    h.op.arg = static_cast<int>(gemv.size());
    h.stage = stage_kind;
    h.bytes = bytes;
    ops.push_back(h);
    gemv.push_back(g);
    return static_cast<int>(gemv.size()) - 1;
  };
  auto res_norm = [&](StepGemv& g, const float* h_in, const float* pending, int pending_parts, const float* norm_w,
                      float* h_out) {
    g.prologue = kPrologueResNorm;
    g.h_in = h_in;
    g.delta = pending;
    g.delta_parts = pending_parts;
    g.delta_stride = c.hidden;
    g.norm_w = norm_w;
    g.eps = c.rms_eps;
    g.h_out = h_out;
    g.normed_out = d->normed;
  };
  // Every product that feeds a residual add writes its (partial) rows here.
  float* out_parts = nullptr;   // allocated below, once max_split is known: patched in afterwards
  {
    HostOp h{};
    h.op.kind = kStepEmbed;
    h.op.items = 1;
    h.stage = GUFO_CUDA_TIMELINE_EMBED;
    ops.push_back(h);
  }
  if (d->embed.type != GUFO_CUDA_Q4_K && d->embed.type != GUFO_CUDA_Q6_K && d->embed.type != GUFO_CUDA_F32) {
    return no("the embedding format runs on the launch chain");
  }
  int cur = 0;
  bool have_pending = false;
  int pending_parts = 1;
  std::vector<int> out_users;    // gemv indices whose y is out_parts
  std::vector<int> out_readers;  // gemv indices whose delta is out_parts
  for (int il = 0; il < c.layers; ++il) {
    auto& l = d->layers[il];
    int gi = product(l.in, -1, false, d->in, GUFO_CUDA_TIMELINE_IN);
    if (gi < 0) {
      return no(problem);
    }
    res_norm(gemv[gi], d->h[cur], have_pending ? reinterpret_cast<const float*>(1) : nullptr, pending_parts,
             l.attn_norm, d->h[cur ^ 1]);
    if (have_pending) {
      out_readers.push_back(gi);
    }
    cur ^= 1;
    if (l.attention) {
      AttnArgs a{c.heads, c.kv_heads, c.head_dim, c.rope_dim, c.max_positions, c.rms_eps, d->position_dev,
                 d->in, l.q_norm, l.k_norm, d->inv_freq, l.keys, l.values, d->queries, d->partials, d->mixed, 0};
      const int items[3] = {c.heads + c.kv_heads, kAttnSplits * c.kv_heads, c.heads};
      const int kinds[3] = {kStepAttnPrep, kStepAttnSlice, kStepAttnMerge};
      for (int k = 0; k < 3; ++k) {
        HostOp h{};
        h.op.kind = kinds[k];
        h.op.items = items[k];
        h.op.arg = static_cast<int>(attn.size());
        h.stage = GUFO_CUDA_TIMELINE_ATTENTION;
        ops.push_back(h);
      }
      attn.push_back(a);
    } else {
      const int dk = l.linear.head_dim;
      if (l.gate_rows.alpha_w == nullptr) {
        return no("ssm_alpha / ssm_beta are not F32 rows");
      }
      if (dk % 32 != 0 || dk > 128 || kSuperBlock % dk != 0 || c.hidden % 4 != 0) {
        return no("the DeltaNet head width does not tile 256-value blocks");
      }
      StepDelta s{};
      s.in = d->in;
      s.gate_x = d->normed;
      s.alpha_w = l.gate_rows.alpha_w;
      s.beta_w = l.gate_rows.beta_w;
      s.cols = c.hidden;
      s.conv_w = l.linear.conv;
      s.ssm_a = l.linear.ssm_a;
      s.dt_bias = l.linear.dt_bias;
      s.conv[0] = l.conv[0];
      s.conv[1] = l.conv[1];
      s.state = l.ssm;
      s.y = d->mixed_raw;
      s.key_heads = l.linear.key_heads;
      s.value_heads = l.linear.value_heads;
      s.head_dim = dk;
      s.conv_kernel = l.linear.conv_kernel;
      HostOp h{};
      h.op.kind = kStepDelta;
      h.op.items = s.value_heads * (dk / 32);
      h.op.arg = static_cast<int>(delta.size());
      h.stage = GUFO_CUDA_TIMELINE_DELTANET;
      h.bytes = 2ll * s.value_heads * dk * dk * 4;
      ops.push_back(h);
      delta.push_back(s);
    }
    gi = product(l.out, -1, true, nullptr, GUFO_CUDA_TIMELINE_OUT);
    if (gi < 0) {
      return no(problem);
    }
    out_users.push_back(gi);
    if (l.attention) {
      gemv[gi].prologue = kProloguePlain;
      gemv[gi].x = d->mixed;
    } else {
      const int64_t channels = static_cast<int64_t>(2 * l.linear.key_heads + l.linear.value_heads) * l.linear.head_dim;
      gemv[gi].prologue = kPrologueGatedNorm;
      gemv[gi].x = d->mixed_raw;
      gemv[gi].z = d->in + channels;
      gemv[gi].gate_w = l.linear.ssm_norm;
      gemv[gi].gate_head_dim = l.linear.head_dim;
      gemv[gi].eps = l.linear.rms_eps;
    }
    const int out_split = gemv[gi].split ? gemv[gi].slabs_per_tile : 1;
    gi = product(l.ffn_in, -1, false, d->ffn, GUFO_CUDA_TIMELINE_FFN_IN);
    if (gi < 0) {
      return no(problem);
    }
    res_norm(gemv[gi], d->h[cur], reinterpret_cast<const float*>(1), out_split, l.post_norm, d->h[cur ^ 1]);
    out_readers.push_back(gi);
    cur ^= 1;
    gi = product(l.ffn_down, -1, true, nullptr, GUFO_CUDA_TIMELINE_FFN_DOWN);
    if (gi < 0) {
      return no(problem);
    }
    out_users.push_back(gi);
    gemv[gi].prologue = kPrologueSwiGlu;
    gemv[gi].x = d->ffn;
    have_pending = true;
    pending_parts = gemv[gi].split ? gemv[gi].slabs_per_tile : 1;
  }
  // The tail: the LM head, or only the final norm.
  const size_t body = ops.size();
  std::vector<HostOp> tail[2];
  for (int with = 0; with < 2; ++with) {
    ops.resize(body);
    const int gi = product(d->lm_head, with ? -1 : 0, false, d->logits, GUFO_CUDA_TIMELINE_LM_HEAD);
    if (gi < 0) {
      return no(problem);
    }
    res_norm(gemv[gi], d->h[cur], have_pending ? reinterpret_cast<const float*>(1) : nullptr, pending_parts,
             d->output_norm, d->h[cur ^ 1]);
    if (have_pending) {
      out_readers.push_back(gi);
    }
    gemv[gi].advance = d->position_dev;
    plan.final_h = d->h[cur ^ 1];
    tail[with].push_back(ops.back());
  }
  ops.resize(body);
  plan.region_bytes = (region + 127) / 128 * 128;
  plan.grid = StepGridBlocks(ctx->device, plan.region_bytes);
  if (plan.grid <= 0) {
    return no("the device cannot hold the kernel's shared memory or has no cooperative launch");
  }
  int rc;
  if ((rc = Alloc(d, static_cast<size_t>(max_split) * c.hidden * 4, reinterpret_cast<void**>(&out_parts))) != GUFO_CUDA_OK) {
    return rc;
  }
  for (int gi : out_users) {
    gemv[gi].y = out_parts;
  }
  for (int gi : out_readers) {
    gemv[gi].delta = out_parts;
  }
  // Items are dealt to the grid's teams in one running round-robin over the
  // whole step, so that a short operation does not always land on the same SMs.
  const int teams = plan.grid * kStepTeams;
  for (int with = 0; with < 2; ++with) {
    std::vector<HostOp> all(ops.begin(), ops.end());
    all.insert(all.end(), tail[with].begin(), tail[with].end());
    std::vector<StepOp> dev;
    int64_t rot = 0;
    for (HostOp& h : all) {
      h.op.rot = static_cast<int>(rot % teams);
      rot += h.op.items;
      dev.push_back(h.op);
      plan.op_stage[with].push_back(h.stage);
      plan.op_bytes[with].push_back(h.bytes);
    }
    plan.nops[with] = static_cast<int>(dev.size());
    if ((rc = Alloc(d, dev.size() * sizeof(StepOp), reinterpret_cast<void**>(&plan.ops[with]))) != GUFO_CUDA_OK) {
      return rc;
    }
    GUFO_CUDA_TRY(cudaMemcpyAsync(plan.ops[with], dev.data(), dev.size() * sizeof(StepOp), cudaMemcpyHostToDevice,
                                  ctx->stream));
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  }
  auto upload = [&](const void* host, size_t bytes, void** dev) -> int {
    const int status = Alloc(d, bytes > 0 ? bytes : 16, dev);
    if (status != GUFO_CUDA_OK) {
      return status;
    }
    if (bytes > 0) {
      GUFO_CUDA_TRY(cudaMemcpyAsync(*dev, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
      GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    }
    return GUFO_CUDA_OK;
  };
  if ((rc = upload(gemv.data(), gemv.size() * sizeof(StepGemv), reinterpret_cast<void**>(&plan.gemv))) != GUFO_CUDA_OK ||
      (rc = upload(delta.data(), delta.size() * sizeof(StepDelta), reinterpret_cast<void**>(&plan.delta))) != GUFO_CUDA_OK ||
      (rc = upload(attn.data(), attn.size() * sizeof(AttnArgs), reinterpret_cast<void**>(&plan.attn))) != GUFO_CUDA_OK ||
      (rc = Alloc(d, 16, reinterpret_cast<void**>(&plan.sync))) != GUFO_CUDA_OK ||
      (rc = Alloc(d, (std::max(plan.nops[0], plan.nops[1]) + 1) * 8, reinterpret_cast<void**>(&plan.stamps))) != GUFO_CUDA_OK) {
    return rc;
  }
  GUFO_CUDA_TRY(cudaMemsetAsync(plan.sync, 0, 16, ctx->stream));
  GUFO_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&plan.error_pinned), 4));
  *plan.error_pinned = 0;
  plan.ok = true;
  return GUFO_CUDA_OK;
}

// Enqueues the one-token step as the persistent kernel.
int EnqueueStepKernel(gufo_cuda_decoder* d, int parity, bool want_logits) {
  auto& plan = d->plan;
  gufo_cuda_ctx* ctx = d->ctx;
  const int with = want_logits ? 1 : 0;
  StepProgram p{};
  p.ops = plan.ops[with];
  p.nops = plan.nops[with];
  p.gemv = plan.gemv;
  p.delta = plan.delta;
  p.attn = plan.attn;
  p.embed = EmbedArgs{d->embed.data, d->embed.type, static_cast<int>(d->embed.row_bytes), d->c.hidden, d->token_dev,
                      d->h[0]};
  p.sync = plan.sync;
  p.stamps = plan.stamps;
  p.parity = parity;
  p.region_bytes = plan.region_bytes;
  int khz = 0;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device);
  p.wait_limit = static_cast<long long>(khz > 0 ? khz : 1000000) * ctx->step_wait_us / 1000;
  p.skip_arrival_at = ctx->step_skip_arrival;
  plan.last_with = with;
  d->final_h = plan.final_h;
  return LaunchStep(ctx, p, plan.grid);
}

// After the stream has been synchronized: a wait of the persistent kernel that
// ran out. Clears the error for the next step.
int CheckStepKernel(gufo_cuda_decoder* d) {
  auto& plan = d->plan;
  if (!plan.ok) {
    return GUFO_CUDA_OK;
  }
  gufo_cuda_ctx* ctx = d->ctx;
  GUFO_CUDA_TRY(cudaMemcpyAsync(plan.error_pinned, plan.sync + 2, 4, cudaMemcpyDeviceToHost, ctx->stream));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  const unsigned code = *plan.error_pinned;
  if (code != 0) {
    GUFO_CUDA_TRY(cudaMemsetAsync(plan.sync, 0, 16, ctx->stream));
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return Fail(GUFO_CUDA_TIMEOUT, "decoder step: a wait inside the step kernel ran out (code " +
                                       std::to_string(code) + "); the outputs and states of that step are invalid");
  }
  return GUFO_CUDA_OK;
}

}  // namespace
}  // namespace gufo

using gufo::Fail;

extern "C" {

int gufo_cuda_matmul_fused_device(gufo_cuda_ctx* ctx, const gufo_cuda_rows* parts, int nparts,
                                  const gufo_cuda_fused_input* in, int tokens, float* y) {
  if (ctx == nullptr || parts == nullptr || in == nullptr || y == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_fused: null pointer");
  }
  if (tokens < 1) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_fused: at least one token");
  }
  gufo::Input input{gufo::kProloguePlain};
  switch (in->prologue) {
    case GUFO_CUDA_PROLOGUE_PLAIN:
    case GUFO_CUDA_PROLOGUE_SWIGLU:
      if (in->x == nullptr || (in->prologue == GUFO_CUDA_PROLOGUE_SWIGLU && in->scratch == nullptr)) {
        return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_fused: x (and, for SwiGLU, scratch) must be given");
      }
      input.prologue = in->prologue == GUFO_CUDA_PROLOGUE_PLAIN ? gufo::kProloguePlain : gufo::kPrologueSwiGlu;
      input.x = in->x;
      break;
    case GUFO_CUDA_PROLOGUE_RES_NORM:
      if (in->residual == nullptr || in->norm_weight == nullptr || in->residual_out == nullptr ||
          in->scratch == nullptr || in->residual_out == in->residual) {
        return Fail(GUFO_CUDA_BAD_ARGUMENT,
                    "matmul_fused: residual, norm_weight, scratch and a residual_out apart from residual");
      }
      input.prologue = gufo::kPrologueResNorm;
      input.h_in = in->residual;
      input.delta = in->delta;
      if (in->delta_parts < 0 || (in->delta_parts > 1 && (in->delta == nullptr || in->delta_stride % 4 != 0))) {
        return Fail(GUFO_CUDA_BAD_ARGUMENT,
                    "matmul_fused: delta_parts vectors need delta and a delta_stride that is a multiple of 4");
      }
      input.delta_parts = in->delta_parts > 1 ? in->delta_parts : 1;
      input.delta_stride = in->delta_stride;
      input.norm_w = in->norm_weight;
      input.h_out = in->residual_out;
      input.advance = in->advance;
      break;
    default:
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_fused: unknown prologue");
  }
  const float* rows[] = {in->x, in->residual, in->delta, in->norm_weight, in->residual_out, in->scratch};
  for (const float* p : rows) {
    if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_fused: rows must be 16-byte aligned");
    }
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::GemvArgs stage;
  const int rc = gufo::BuildGemvArgs(ctx, parts, nparts, &stage);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  if (stage.cols % 4 != 0) {
    return Fail(GUFO_CUDA_SHAPE, "matmul_fused: cols must be a multiple of 4");
  }
  bool activate = false;
  if (in->epilogue == GUFO_CUDA_EPILOGUE_SWIGLU) {
    if (!gufo::SwiGluInProduct(ctx, stage, tokens)) {
      return Fail(GUFO_CUDA_UNSUPPORTED_TYPE, "matmul_fused: this product cannot activate its own rows");
    }
    activate = true;
  } else if (in->epilogue != GUFO_CUDA_EPILOGUE_NONE) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_fused: unknown epilogue");
  }
  return gufo::FusedProduct(ctx, in->rms_eps, stage, input, in->scratch, y, tokens, nullptr, nullptr, activate);
}

// The fused input of the peer-group products, checked.
static int PeerProductInput(const gufo_cuda_fused_input* in, const char* who, gufo::Input* input) {
  *input = gufo::Input{gufo::kProloguePlain};
  switch (in->prologue) {
    case GUFO_CUDA_PROLOGUE_PLAIN:
    case GUFO_CUDA_PROLOGUE_SWIGLU:
      if (in->x == nullptr) {
        return Fail(GUFO_CUDA_BAD_ARGUMENT, std::string(who) + ": x must be given");
      }
      input->prologue = in->prologue == GUFO_CUDA_PROLOGUE_PLAIN ? gufo::kProloguePlain : gufo::kPrologueSwiGlu;
      input->x = in->x;
      break;
    case GUFO_CUDA_PROLOGUE_RES_NORM:
      if (in->residual == nullptr || in->norm_weight == nullptr || in->residual_out == nullptr ||
          in->scratch == nullptr || in->residual_out == in->residual) {
        return Fail(GUFO_CUDA_BAD_ARGUMENT,
                    std::string(who) + ": residual, norm_weight, scratch and a residual_out apart from residual");
      }
      if (in->delta_parts < 0 || (in->delta_parts > 1 && (in->delta == nullptr || in->delta_stride % 4 != 0))) {
        return Fail(GUFO_CUDA_BAD_ARGUMENT,
                    std::string(who) + ": delta_parts vectors need delta and a delta_stride that is a multiple of 4");
      }
      input->prologue = gufo::kPrologueResNorm;
      input->h_in = in->residual;
      input->delta = in->delta;
      input->delta_parts = in->delta_parts > 1 ? in->delta_parts : 1;
      input->delta_stride = in->delta_stride;
      input->norm_w = in->norm_weight;
      input->h_out = in->residual_out;
      input->advance = in->advance;
      break;
    default:
      return Fail(GUFO_CUDA_BAD_ARGUMENT, std::string(who) + ": unknown prologue");
  }
  const float* rows[] = {in->x, in->residual, in->delta, in->norm_weight, in->residual_out, in->scratch};
  for (const float* p : rows) {
    if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, std::string(who) + ": rows must be 16-byte aligned");
    }
  }
  return GUFO_CUDA_OK;
}

static gufo::PeerWait WaitOn(const gufo_cuda_peer_group* g, int wait_slot) {
  gufo::PeerWait wait{};
  wait.header = reinterpret_cast<const unsigned*>(g->arena[g->rank]);
  wait.world = g->world;
  wait.slot = wait_slot;
  wait.limit = g->limit;
  return wait;
}

int gufo_cuda_matmul_gather_device(gufo_cuda_peer_group* g, const gufo_cuda_rows* parts, int nparts,
                                   const gufo_cuda_fused_input* in, size_t arena_offset, int slot, int wait_slot) {
  if (g == nullptr || parts == nullptr || in == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_gather: null pointer");
  }
  if (slot < 0 || slot >= gufo::kPeerSlots || wait_slot >= gufo::kPeerSlots) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_gather: slots are 0 to 7 (wait_slot < 0: no wait)");
  }
  if (in->epilogue != GUFO_CUDA_EPILOGUE_NONE) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_gather: rows that travel to the peers are stored as they are");
  }
  gufo::Input input{gufo::kProloguePlain};
  int rc = PeerProductInput(in, "matmul_gather", &input);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  gufo_cuda_ctx* ctx = g->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::GemvArgs stage;
  rc = gufo::BuildGemvArgs(ctx, parts, nparts, &stage);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  if (stage.cols % 4 != 0) {
    return Fail(GUFO_CUDA_SHAPE, "matmul_gather: cols must be a multiple of 4");
  }
  const size_t local = static_cast<size_t>(stage.total_rows);
  if (arena_offset < GUFO_CUDA_PEER_HEADER_BYTES || arena_offset % 16 != 0 ||
      arena_offset + local * 4 * g->world > g->arena_bytes) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_gather: the full vector must lie inside the arena, 16-byte aligned");
  }
  gufo::PeerOut out{};
  out.world = g->world;
  out.rank = g->rank;
  out.slot = slot;
  for (int p = 0; p < g->world; ++p) {
    out.y[p] = reinterpret_cast<float*>(g->arena[p] + arena_offset) + static_cast<size_t>(g->rank) * local;
    out.header[p] = reinterpret_cast<unsigned*>(g->arena[p]);
  }
  const gufo::PeerWait wait = WaitOn(g, wait_slot);
  return gufo::FusedProduct(ctx, in->rms_eps, stage, input, in->scratch, out.y[g->rank], 1, &out,
                            wait_slot >= 0 ? &wait : nullptr);
}

int gufo_cuda_matmul_wait_device(gufo_cuda_peer_group* g, const gufo_cuda_rows* parts, int nparts,
                                 const gufo_cuda_fused_input* in, int wait_slot, float* device_y) {
  if (g == nullptr || parts == nullptr || in == nullptr || device_y == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_wait: null pointer");
  }
  if (wait_slot < 0 || wait_slot >= gufo::kPeerSlots || (reinterpret_cast<uintptr_t>(device_y) & 15) != 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_wait: wait_slot is 0 to 7 and y 16-byte aligned");
  }
  gufo::Input input{gufo::kProloguePlain};
  int rc = PeerProductInput(in, "matmul_wait", &input);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  gufo_cuda_ctx* ctx = g->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::GemvArgs stage;
  rc = gufo::BuildGemvArgs(ctx, parts, nparts, &stage);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  if (stage.cols % 4 != 0) {
    return Fail(GUFO_CUDA_SHAPE, "matmul_wait: cols must be a multiple of 4");
  }
  bool activate = false;
  if (in->epilogue == GUFO_CUDA_EPILOGUE_SWIGLU) {
    if (!gufo::SwiGluInProduct(ctx, stage, 1)) {
      return Fail(GUFO_CUDA_UNSUPPORTED_TYPE, "matmul_wait: this product cannot activate its own rows");
    }
    activate = true;
  } else if (in->epilogue != GUFO_CUDA_EPILOGUE_NONE) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_wait: unknown epilogue");
  }
  const gufo::PeerWait wait = WaitOn(g, wait_slot);
  return gufo::FusedProduct(ctx, in->rms_eps, stage, input, in->scratch, device_y, 1, nullptr, &wait, activate);
}

int gufo_cuda_decoder_create(gufo_cuda_ctx* ctx, const gufo_cuda_decoder_config* config,
                             const gufo_cuda_decoder_weights* weights, gufo_cuda_decoder** out) {
  if (ctx == nullptr || config == nullptr || weights == nullptr || out == nullptr ||
      weights->layers == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_create: null pointer");
  }
  *out = nullptr;
  const gufo_cuda_decoder_config& c = *config;
  if (c.layers <= 0 || c.hidden <= 0 || c.ffn <= 0 || c.vocab <= 0 || c.full_attention_interval <= 0 ||
      c.kv_heads <= 0 || c.heads % c.kv_heads != 0 || c.heads / c.kv_heads > gufo::kMaxGroup ||
      c.head_dim % 32 != 0 || c.head_dim > 32 * gufo::kMaxPerLane || c.rope_dim > c.head_dim ||
      c.rope_dim % 2 != 0 || c.max_positions <= 0 || c.hidden % 256 != 0 || c.experts < 0 ||
      (c.experts > 0 && (c.experts_used <= 0 || c.experts_used > c.experts || c.expert_ffn <= 0 ||
                         c.expert_ffn % 256 != 0))) {
    return Fail(GUFO_CUDA_SHAPE, "decoder_create: unsupported or inconsistent shape");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  auto* d = new gufo_cuda_decoder();
  d->ctx = ctx;
  d->c = c;
  auto fail = [&](int rc) {
    gufo_cuda_decoder_destroy(d);
    return rc;
  };
  const int64_t key_dim = static_cast<int64_t>(c.linear_key_heads) * c.linear_head_dim;
  const int64_t value_dim = static_cast<int64_t>(c.linear_value_heads) * c.linear_head_dim;
  const int64_t channels = 2 * key_dim + value_dim;
  const int64_t attn_dim = static_cast<int64_t>(c.heads) * c.head_dim;
  const int64_t kv_dim = static_cast<int64_t>(c.kv_heads) * c.head_dim;
  int rc;
  const gufo::Matrix* embed = ctx->FindMatrix(weights->token_embd);
  if (embed == nullptr || embed->cols != c.hidden || embed->rows != c.vocab) {
    return fail(Fail(GUFO_CUDA_SHAPE, "decoder_create: token_embd must be [hidden, vocab]"));
  }
  if (embed->type != GUFO_CUDA_Q4_K && embed->type != GUFO_CUDA_Q6_K && embed->type != GUFO_CUDA_F32) {
    return fail(Fail(GUFO_CUDA_UNSUPPORTED_TYPE, "decoder_create: token_embd must be Q4_K, Q6_K or F32 here"));
  }
  d->embed = *embed;
  {
    const gufo_cuda_matrix head = weights->output != 0 ? weights->output : weights->token_embd;
    const int64_t rows = c.vocab;
    if ((rc = gufo::Stack(ctx, &head, &rows, 1, c.hidden, "the LM head", &d->lm_head)) != GUFO_CUDA_OK) {
      return fail(rc);
    }
    // One launch of the tensor-core GEMV: its stores can mirror the logits into host memory.
    const int type = d->lm_head.parts[0].type;
    d->mirror_ok = d->lm_head.nparts == 1 &&
                   ((type == GUFO_CUDA_Q4_K && gufo::Q4KFastFits(c.hidden, 1)) ||
                    (type == GUFO_CUDA_Q6_K && gufo::Q6KFastFits(c.hidden, 1)));
  }
  if ((rc = gufo::UploadVec(d, weights->output_norm, c.hidden, &d->output_norm, "output_norm")) != GUFO_CUDA_OK) {
    return fail(rc);
  }
  size_t in_max = 0;
  int linear_layers = 0;
  d->layers.resize(c.layers);
  for (int il = 0; il < c.layers; ++il) {
    const gufo_cuda_layer_weights& w = weights->layers[il];
    auto& l = d->layers[il];
    l.attention = (il + 1) % c.full_attention_interval == 0;
    if ((rc = gufo::UploadVec(d, w.attn_norm, c.hidden, &l.attn_norm, "attn_norm")) != GUFO_CUDA_OK ||
        (rc = gufo::UploadVec(d, w.post_attention_norm, c.hidden, &l.post_norm, "post_attention_norm")) !=
            GUFO_CUDA_OK) {
      return fail(rc);
    }
    if (l.attention) {
      const gufo_cuda_matrix in[3] = {w.attn_q, w.attn_k, w.attn_v};
      const int64_t rows[3] = {2 * attn_dim, kv_dim, kv_dim};
      if ((rc = gufo::Stack(ctx, in, rows, 3, c.hidden, "attn_q/k/v", &l.in)) != GUFO_CUDA_OK) {
        return fail(rc);
      }
      const int64_t out_rows = c.hidden;
      if ((rc = gufo::Stack(ctx, &w.attn_output, &out_rows, 1, attn_dim, "attn_output", &l.out)) != GUFO_CUDA_OK ||
          (rc = gufo::UploadVec(d, w.attn_q_norm, c.head_dim, &l.q_norm, "attn_q_norm")) != GUFO_CUDA_OK ||
          (rc = gufo::UploadVec(d, w.attn_k_norm, c.head_dim, &l.k_norm, "attn_k_norm")) != GUFO_CUDA_OK) {
        return fail(rc);
      }
      const size_t cache = static_cast<size_t>(c.max_positions) * kv_dim * sizeof(__half);
      if ((rc = gufo::Alloc(d, cache, reinterpret_cast<void**>(&l.keys))) != GUFO_CUDA_OK ||
          (rc = gufo::Alloc(d, cache, reinterpret_cast<void**>(&l.values))) != GUFO_CUDA_OK) {
        return fail(rc);
      }
    } else {
      if (c.linear_head_dim % 32 != 0 || c.linear_head_dim > 128 || c.linear_key_heads <= 0 ||
          c.linear_value_heads % c.linear_key_heads != 0 || c.conv_kernel < 2 || c.conv_kernel > 8) {
        return fail(Fail(GUFO_CUDA_SHAPE, "decoder_create: unsupported DeltaNet shape"));
      }
      const gufo_cuda_matrix in[4] = {w.attn_qkv, w.attn_gate, w.ssm_alpha, w.ssm_beta};
      const int64_t rows[4] = {channels, value_dim, c.linear_value_heads, c.linear_value_heads};
      if ((rc = gufo::Stack(ctx, in, rows, 4, c.hidden, "attn_qkv/gate/ssm_alpha/ssm_beta", &l.in)) != GUFO_CUDA_OK) {
        return fail(rc);
      }
      // F32 alpha / beta rows (the usual case) are multiplied inside the mixer
      // kernel: the input product then stops after [qkv | z], one launch less.
      const gufo::Matrix* alpha = ctx->FindMatrix(w.ssm_alpha);
      const gufo::Matrix* beta = ctx->FindMatrix(w.ssm_beta);
      if (alpha->type == GUFO_CUDA_F32 && beta->type == GUFO_CUDA_F32 && c.hidden % 4 == 0) {
        if ((rc = gufo::Stack(ctx, in, rows, 2, c.hidden, "attn_qkv/gate", &l.in)) != GUFO_CUDA_OK) {
          return fail(rc);
        }
        l.gate_rows.alpha_w = reinterpret_cast<const float*>(alpha->data);
        l.gate_rows.beta_w = reinterpret_cast<const float*>(beta->data);
        l.gate_rows.cols = c.hidden;
      }
      const int64_t out_rows = c.hidden;
      if ((rc = gufo::Stack(ctx, &w.ssm_out, &out_rows, 1, value_dim, "ssm_out", &l.out)) != GUFO_CUDA_OK) {
        return fail(rc);
      }
      l.linear.key_heads = c.linear_key_heads;
      l.linear.value_heads = c.linear_value_heads;
      l.linear.head_dim = c.linear_head_dim;
      l.linear.conv_kernel = c.conv_kernel;
      l.linear.rms_eps = c.rms_eps;
      if ((rc = gufo::UploadVec(d, w.ssm_conv1d, channels * c.conv_kernel, &l.linear.conv, "ssm_conv1d")) != GUFO_CUDA_OK ||
          (rc = gufo::UploadVec(d, w.ssm_a, c.linear_value_heads, &l.linear.ssm_a, "ssm_a")) != GUFO_CUDA_OK ||
          (rc = gufo::UploadVec(d, w.ssm_dt_bias, c.linear_value_heads, &l.linear.dt_bias, "ssm_dt.bias")) != GUFO_CUDA_OK ||
          (rc = gufo::UploadVec(d, w.ssm_norm, c.linear_head_dim, &l.linear.ssm_norm, "ssm_norm")) != GUFO_CUDA_OK) {
        return fail(rc);
      }
      ++linear_layers;
    }
    const gufo_cuda_matrix gate_up[2] = {w.ffn_gate, w.ffn_up};
    const int64_t ffn_rows[2] = {c.ffn, c.ffn};
    const int64_t down_rows = c.hidden;
    if ((rc = gufo::Stack(ctx, gate_up, ffn_rows, 2, c.hidden, "ffn_gate/up", &l.ffn_in)) != GUFO_CUDA_OK ||
        (rc = gufo::Stack(ctx, &w.ffn_down, &down_rows, 1, c.ffn, "ffn_down", &l.ffn_down)) != GUFO_CUDA_OK) {
      return fail(rc);
    }
    if (c.experts > 0) {
      const gufo_cuda_matrix router[2] = {w.ffn_gate_inp, w.ffn_gate_inp_shexp};
      const int64_t router_rows[2] = {c.experts, 1};
      const gufo_cuda_expert_bank bank{w.ffn_gate_exps, w.ffn_up_exps, w.ffn_down_exps, c.experts, c.expert_ffn,
                                       c.hidden};
      if ((rc = gufo::Stack(ctx, router, router_rows, 2, c.hidden, "ffn_gate_inp/ffn_gate_inp_shexp", &l.router)) !=
              GUFO_CUDA_OK ||
          (rc = gufo::BuildExpertBank(ctx, bank, &l.bank)) != GUFO_CUDA_OK) {
        return fail(rc);
      }
    }
    in_max = std::max(in_max, static_cast<size_t>(l.in.total_rows));
  }
  // The DeltaNet layers' windows and states: one allocation per kind.
  {
    const size_t conv_floats = static_cast<size_t>(c.conv_kernel - 1) * channels;
    const size_t ssm_floats = static_cast<size_t>(value_dim) * c.linear_head_dim;
    d->conv_all_bytes = conv_floats * 4 * linear_layers;
    d->ssm_all_bytes = ssm_floats * 4 * linear_layers;
    if (linear_layers > 0) {
      for (float*& block : d->conv_all) {
        if ((rc = gufo::Alloc(d, d->conv_all_bytes, reinterpret_cast<void**>(&block))) != GUFO_CUDA_OK) {
          return fail(rc);
        }
      }
      for (float*& block : d->ssm_all) {
        if ((rc = gufo::Alloc(d, d->ssm_all_bytes, reinterpret_cast<void**>(&block))) != GUFO_CUDA_OK) {
          return fail(rc);
        }
      }
    }
    size_t at = 0;
    for (auto& l : d->layers) {
      if (l.attention) {
        continue;
      }
      l.conv[0] = d->conv_all[0] + at * conv_floats;
      l.conv[1] = d->conv_all[1] + at * conv_floats;
      l.conv_saved = d->conv_all[2] + at * conv_floats;
      l.ssm = d->ssm_all[0] + at * ssm_floats;
      l.ssm_spec = d->ssm_all[1] + at * ssm_floats;
      ++at;
    }
  }
  std::vector<float> inv_freq(c.rope_dim / 2 > 0 ? c.rope_dim / 2 : 1);
  for (int i = 0; i < c.rope_dim / 2; ++i) {
    // The reference's table (decoder.cpp:85-90).
    inv_freq[i] = static_cast<float>(
        1.0 / std::pow(static_cast<double>(c.rope_theta), 2.0 * i / static_cast<double>(c.rope_dim)));
  }
  if ((rc = gufo::UploadVec(d, inv_freq.data(), inv_freq.size(), &d->inv_freq, "rope")) != GUFO_CUDA_OK) {
    return fail(rc);
  }
  const size_t mixed = static_cast<size_t>(std::max<int64_t>(value_dim, attn_dim));
  const int group = c.heads / c.kv_heads;
  // Activations for the two rows of a pair step; a one-token step uses the first.
  const size_t two = gufo::kStepTokens;
  struct Buf {
    float** p;
    size_t n;
  } bufs[] = {{&d->h[0], two * c.hidden}, {&d->h[1], two * c.hidden},
              {&d->normed, two * c.hidden},
              {&d->in, two * in_max}, {&d->mixed, two * mixed}, {&d->mixed_raw, two * mixed},
              {&d->out, two * c.hidden},
              {&d->ffn, two * 2 * c.ffn}, {&d->act, two * c.ffn},
              {&d->logits, two * c.vocab}, {&d->queries, static_cast<size_t>(attn_dim)},
              {&d->partials, static_cast<size_t>(c.kv_heads) * gufo::kAttnSplits * group * (c.head_dim + 2)},
              // MoE scratch (a few floats for a dense model).
              {&d->router, two * (static_cast<size_t>(c.experts) + 1)},
              {&d->route_weights, two * c.experts_used + 1},
              {&d->shared_scale, two},
              {&d->expert_ffn, two * c.experts_used * 2 * c.expert_ffn + 1},
              {&d->expert_act, two * c.experts_used * c.expert_ffn + 1},
              {&d->expert_out, two * c.experts_used * c.hidden + 1}};
  for (auto& b : bufs) {
    if ((rc = gufo::Alloc(d, b.n * 4, reinterpret_cast<void**>(b.p))) != GUFO_CUDA_OK) {
      return fail(rc);
    }
  }
  if ((rc = gufo::Alloc(d, 4 * (two * c.experts_used + 1), reinterpret_cast<void**>(&d->chosen))) != GUFO_CUDA_OK ||
      (rc = gufo::Alloc(d, 4, reinterpret_cast<void**>(&d->position_dev))) != GUFO_CUDA_OK ||
      (rc = gufo::Alloc(d, 4 * two, reinterpret_cast<void**>(&d->token_dev))) != GUFO_CUDA_OK) {
    return fail(rc);
  }
  cudaError_t e = cudaMallocHost(reinterpret_cast<void**>(&d->token_pinned), 4 * two * (gufo::kTokenSlots + 1));
  if (e != cudaSuccess) {
    return fail(gufo::CudaFail(e, "cudaMallocHost"));
  }
  for (cudaEvent_t& read : d->token_read) {
    if ((e = cudaEventCreateWithFlags(&read, cudaEventDisableTiming)) != cudaSuccess) {
      return fail(gufo::CudaFail(e, "cudaEventCreate"));
    }
  }
  if ((rc = gufo::BuildStepPlan(d)) != GUFO_CUDA_OK) {
    return fail(rc);
  }
  *out = d;
  // Zero states (the lock is already held: reset's body inline).
  if (d->conv_all_bytes > 0) {
    cudaMemsetAsync(d->conv_all[0], 0, d->conv_all_bytes, ctx->stream);
    cudaMemsetAsync(d->conv_all[1], 0, d->conv_all_bytes, ctx->stream);
    cudaMemsetAsync(d->ssm_all[0], 0, d->ssm_all_bytes, ctx->stream);
  }
  cudaMemsetAsync(d->position_dev, 0, 4, ctx->stream);
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  return GUFO_CUDA_OK;
}

int gufo_cuda_decoder_destroy(gufo_cuda_decoder* d) {
  if (d == nullptr) {
    return GUFO_CUDA_OK;
  }
  cudaSetDevice(d->ctx->device);
  cudaStreamSynchronize(d->ctx->stream);
  for (auto& per_count : d->graph) {
    for (auto& per_window : per_count) {
      for (cudaGraphExec_t g : per_window) {
        if (g != nullptr) {
          cudaGraphExecDestroy(g);
        }
      }
    }
  }
  for (void* p : d->owned) {
    cudaFree(p);
  }
  for (cudaEvent_t e : d->marks) {
    cudaEventDestroy(e);
  }
  if (d->token_pinned != nullptr) {
    cudaFreeHost(d->token_pinned);
  }
  if (d->plan.error_pinned != nullptr) {
    cudaFreeHost(d->plan.error_pinned);
  }
  for (cudaEvent_t read : d->token_read) {
    if (read != nullptr) {
      cudaEventDestroy(read);
    }
  }
  delete d;
  return GUFO_CUDA_OK;
}

int gufo_cuda_decoder_reset(gufo_cuda_decoder* d) {
  if (d == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_reset: null decoder");
  }
  gufo_cuda_ctx* ctx = d->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  if (d->conv_all_bytes > 0) {
    GUFO_CUDA_TRY(cudaMemsetAsync(d->conv_all[0], 0, d->conv_all_bytes, ctx->stream));
    GUFO_CUDA_TRY(cudaMemsetAsync(d->conv_all[1], 0, d->conv_all_bytes, ctx->stream));
    GUFO_CUDA_TRY(cudaMemsetAsync(d->ssm_all[0], 0, d->ssm_all_bytes, ctx->stream));
  }
  GUFO_CUDA_TRY(cudaMemsetAsync(d->position_dev, 0, 4, ctx->stream));
  d->position = 0;
  d->conv_cur = 0;
  d->pending = 0;
  return GUFO_CUDA_OK;
}

int gufo_cuda_decoder_step_tokens(gufo_cuda_decoder* d, const int* tokens, int count, int want_logits,
                                  float* host_logits) {
  if (d == nullptr || tokens == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_step: null pointer");
  }
  if (count < 1 || count > gufo::kStepTokens) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_step: 1 or 2 tokens per step");
  }
  for (int t = 0; t < count; ++t) {
    if (tokens[t] < 0 || tokens[t] >= d->c.vocab) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "qwen35: token id out of range");
    }
  }
  if (d->pending != 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_step: the last two-token step awaits decoder_resolve");
  }
  if (d->position + count > d->c.max_positions) {
    return Fail(GUFO_CUDA_TOO_LARGE, "decoder_step: the attention cache is full");
  }
  if (host_logits != nullptr && want_logits == 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_step: logits asked for and switched off");
  }
  gufo_cuda_ctx* ctx = d->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  {
    const unsigned slot = d->token_slot++ % gufo::kTokenSlots;
    int* staged = d->token_pinned + slot * gufo::kStepTokens;
    GUFO_CUDA_TRY(cudaEventSynchronize(d->token_read[slot]));   // returns at once for a slot never used
    for (int t = 0; t < count; ++t) {
      staged[t] = tokens[t];
    }
    GUFO_CUDA_TRY(cudaMemcpyAsync(d->token_dev, staged, 4 * count, cudaMemcpyHostToDevice, ctx->stream));
    GUFO_CUDA_TRY(cudaEventRecord(d->token_read[slot], ctx->stream));
  }
  const int parity = d->conv_cur;
  const int pair = count - 1;
  int with = want_logits != 0 ? 1 : 0;
  // One token into a pinned host buffer that the device can address: the LM
  // head mirrors its rows there and no copy follows.
  if (host_logits != nullptr && count == 1 && d->mirror_ok && d->c.use_graph && !d->timeline && !ctx->force_general &&
      !ctx->step_kernel && d->eager_runs[pair][1] >= 2) {
    if (host_logits != d->host_mirror_for) {
      cudaPointerAttributes attr{};
      float* device_side = nullptr;
      if (cudaPointerGetAttributes(&attr, host_logits) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
          attr.devicePointer != nullptr && (reinterpret_cast<uintptr_t>(attr.devicePointer) & 15) == 0) {
        device_side = static_cast<float*>(attr.devicePointer);
      } else {
        cudaGetLastError();   // pageable memory is not an error here
      }
      // The graphs of the old buffer hold its address.
      for (int w = 0; w < 2; ++w) {
        if (d->graph[0][w][2] != nullptr) {
          cudaGraphExecDestroy(d->graph[0][w][2]);
          d->graph[0][w][2] = nullptr;
        }
      }
      d->host_mirror = device_side;
      d->host_mirror_for = host_logits;
    }
    if (d->host_mirror != nullptr) {
      with = 2;
    }
  }
  const int ran = with == 2 ? 1 : with;   // which count of eager runs the step belongs to
  auto enqueue = [&]() { return gufo::EnqueueStep(d, parity, with != 0, count, with == 2); };
  // One token: the whole step as one persistent kernel, where the model allows it.
  const bool kernel_step = count == 1 && d->plan.ok && ctx->step_kernel && !ctx->force_general && !d->timeline;
  if (kernel_step) {
    const int rc = gufo::EnqueueStepKernel(d, parity, with != 0);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
  } else if (d->c.use_graph && d->eager_runs[pair][ran] >= 2 && !d->timeline) {
    cudaGraphExec_t& exec = d->graph[pair][parity][with];
    if (exec == nullptr) {
      cudaGraph_t graph = nullptr;
      GUFO_CUDA_TRY(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
      const int64_t before = ctx->launches.load();
      const int rc = enqueue();
      d->graph_kernels[pair][parity][with] = ctx->launches.load() - before;
      ctx->launches.store(before);   // counted at every replay instead
      const cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
      if (rc != GUFO_CUDA_OK || e != cudaSuccess) {
        if (graph != nullptr) {
          cudaGraphDestroy(graph);
        }
        return rc != GUFO_CUDA_OK ? rc : gufo::CudaFail(e, "cudaStreamEndCapture");
      }
      const cudaError_t ei = cudaGraphInstantiate(&exec, graph, 0);
      cudaGraphDestroy(graph);
      if (ei != cudaSuccess) {
        exec = nullptr;
        return gufo::CudaFail(ei, "cudaGraphInstantiate");
      }
    }
    GUFO_CUDA_TRY(cudaGraphLaunch(exec, ctx->stream));
    ctx->launches.fetch_add(d->graph_kernels[pair][parity][with]);
  } else {
    const int rc = enqueue();
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
    ++d->eager_runs[pair][ran];
  }
  d->position += count;
  d->conv_cur ^= 1;
  d->pending = count == 2 ? 2 : 0;
  ++d->steps;
  if (d->timeline) {
    // Fold this step's marks into the per-stage totals.
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    for (size_t i = 1; i < d->mark_kind.size(); ++i) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, d->marks[i - 1], d->marks[i]);
      if (d->mark_kind[i] >= 0) {
        d->stage_ms[d->mark_kind[i]] += ms;
      }
    }
    d->mark_kind.clear();
    ++d->timeline_steps;
  }
  if (host_logits != nullptr && with == 2) {
    // The LM head wrote the caller's buffer itself; the step's end is all there is to wait for.
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  } else if (host_logits != nullptr) {
    GUFO_CUDA_TRY(cudaMemcpyAsync(host_logits, d->logits, static_cast<size_t>(count) * d->c.vocab * 4,
                                  cudaMemcpyDeviceToHost, ctx->stream));
    if (kernel_step) {
      return gufo::CheckStepKernel(d);   // copies the error word down and waits for the stream
    }
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  }
  return GUFO_CUDA_OK;
}

int gufo_cuda_decoder_status(gufo_cuda_decoder* d) {
  if (d == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_status: null decoder");
  }
  gufo_cuda_ctx* ctx = d->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  return gufo::CheckStepKernel(d);
}

int gufo_cuda_decoder_step_profile(gufo_cuda_decoder* d, int capacity, int* stages, int64_t* bytes, double* us,
                                   int* count) {
  if (d == nullptr || count == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_step_profile: null pointer");
  }
  *count = 0;
  const auto& plan = d->plan;
  if (!plan.ok) {
    return GUFO_CUDA_OK;   // the model runs on the launch chain: no operations to report
  }
  gufo_cuda_ctx* ctx = d->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  const int with = plan.last_with;
  const int n = plan.nops[with];
  std::vector<unsigned long long> stamps(n + 1);
  GUFO_CUDA_TRY(cudaMemcpyAsync(stamps.data(), plan.stamps, (n + 1) * 8, cudaMemcpyDeviceToHost, ctx->stream));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  *count = n;
  for (int i = 0; i < n && i < capacity; ++i) {
    if (stages != nullptr) {
      stages[i] = plan.op_stage[with][i];
    }
    if (bytes != nullptr) {
      bytes[i] = plan.op_bytes[with][i];
    }
    if (us != nullptr) {
      us[i] = static_cast<double>(stamps[i + 1] - stamps[i]) * 1e-3;
    }
  }
  return GUFO_CUDA_OK;
}

int gufo_cuda_decoder_step(gufo_cuda_decoder* d, int token, float* host_logits) {
  return gufo_cuda_decoder_step_tokens(d, &token, 1, 1, host_logits);
}

int gufo_cuda_decoder_resolve(gufo_cuda_decoder* d, int keep_second) {
  if (d == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_resolve: null decoder");
  }
  if (d->pending != 2) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_resolve: the last step was not a two-token step");
  }
  gufo_cuda_ctx* ctx = d->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  if (keep_second != 0) {
    // The draft's states become the states (ssm <-> ssm_spec in the reference).
    if (d->ssm_all_bytes > 0) {
      GUFO_CUDA_TRY(cudaMemcpyAsync(d->ssm_all[0], d->ssm_all[1], d->ssm_all_bytes, cudaMemcpyDeviceToDevice,
                                    ctx->stream));
    }
  } else {
    // Back to just after the first token: its conv windows, one position less;
    // the second token's cache rows are overwritten by the next step.
    if (d->conv_all_bytes > 0) {
      GUFO_CUDA_TRY(cudaMemcpyAsync(d->conv_all[d->conv_cur], d->conv_all[2], d->conv_all_bytes,
                                    cudaMemcpyDeviceToDevice, ctx->stream));
    }
    --d->position;
    int* word = d->token_pinned + gufo::kTokenSlots * gufo::kStepTokens;
    *word = d->position;
    GUFO_CUDA_TRY(cudaMemcpyAsync(d->position_dev, word, 4, cudaMemcpyHostToDevice, ctx->stream));
    // The pinned word is read when the copy runs: wait, so that a later
    // Resolve cannot overwrite it first.
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  }
  d->pending = 0;
  return GUFO_CUDA_OK;
}

int gufo_cuda_decoder_hidden_device(gufo_cuda_decoder* d, int t, const float** hidden) {
  if (d == nullptr || hidden == nullptr || t < 0 || t >= gufo::kStepTokens || d->final_h == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_hidden_device: no such row");
  }
  *hidden = d->final_h + static_cast<size_t>(t) * d->c.hidden;
  return GUFO_CUDA_OK;
}

int gufo_cuda_decoder_logits_device(gufo_cuda_decoder* d, const float** device_logits) {
  if (d == nullptr || device_logits == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_logits_device: null pointer");
  }
  *device_logits = d->logits;
  return GUFO_CUDA_OK;
}

int gufo_cuda_decoder_timeline(gufo_cuda_decoder* d, int enable, double* stage_ms, int* steps) {
  if (d == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_timeline: null decoder");
  }
  std::lock_guard<std::mutex> lock(d->ctx->mu);
  if (stage_ms != nullptr) {
    for (int k = 0; k < GUFO_CUDA_TIMELINE_KINDS; ++k) {
      stage_ms[k] = d->stage_ms[k];
    }
  }
  if (steps != nullptr) {
    *steps = d->timeline_steps;
  }
  if ((enable != 0) != d->timeline) {
    d->timeline = enable != 0;
    for (double& v : d->stage_ms) {
      v = 0;
    }
    d->timeline_steps = 0;
  }
  return GUFO_CUDA_OK;
}

int gufo_cuda_decoder_position(const gufo_cuda_decoder* d) { return d == nullptr ? -1 : d->position; }

int gufo_cuda_decoder_linear_state(gufo_cuda_decoder* d, int layer, float* host_conv, float* host_ssm) {
  if (d == nullptr || layer < 0 || layer >= static_cast<int>(d->layers.size()) || d->layers[layer].attention) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "decoder_linear_state: not a DeltaNet layer");
  }
  gufo_cuda_ctx* ctx = d->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  const gufo_cuda_decoder_config& c = d->c;
  const auto& l = d->layers[layer];
  const size_t channels = static_cast<size_t>(2 * c.linear_key_heads + c.linear_value_heads) * c.linear_head_dim;
  if (host_conv != nullptr) {
    GUFO_CUDA_TRY(cudaMemcpyAsync(host_conv, l.conv[d->conv_cur], (c.conv_kernel - 1) * channels * 4,
                                  cudaMemcpyDeviceToHost, ctx->stream));
  }
  if (host_ssm != nullptr) {
    GUFO_CUDA_TRY(cudaMemcpyAsync(host_ssm, l.ssm, static_cast<size_t>(c.linear_value_heads) * c.linear_head_dim *
                                                       c.linear_head_dim * 4, cudaMemcpyDeviceToHost, ctx->stream));
  }
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  return GUFO_CUDA_OK;
}

}  // extern "C"
