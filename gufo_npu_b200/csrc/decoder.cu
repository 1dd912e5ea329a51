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

#include "gemv.cuh"
#include "moe.cuh"

namespace gufo {
namespace {

constexpr int kSmallThreads = 256;
constexpr int kAttnSplits = 8;      // position slices per KV head
constexpr int kMaxGroup = 8;        // query heads per KV head
constexpr int kMaxPerLane = 8;      // head_dim / 32
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

// h = dequantized row *token of the embedding matrix (quant::Dequantize of one
// row, src/models/qwen35/decoder.cpp:486-489). One thread block.
struct EmbedArgs {
  const uint8_t* data;
  int type;
  int row_bytes;
  int cols;
  const int* token;
  float* h;
};

__global__ void __launch_bounds__(kSmallThreads)
EmbedKernel(const __grid_constant__ EmbedArgs a) {
  GridLaunchDependents();
  GridDependencyWait();
  const uint8_t* row = a.data + static_cast<size_t>(*a.token) * a.row_bytes;
  const int blocks = a.cols / kSuperBlock;
  if (a.type == GUFO_CUDA_Q4_K) {
    for (int item = threadIdx.x; item < blocks * 32; item += kSmallThreads) {
      const int b = item >> 5, word = item & 31, p = word >> 3, c = word & 7;
      const uint32_t* block = reinterpret_cast<const uint32_t*>(row + b * kQ4KBytes);
      const uint32_t dd = block[0];
      const float d = HalfBitsToFloat(static_cast<uint16_t>(dd & 0xFFFF));
      const float dmin = HalfBitsToFloat(static_cast<uint16_t>(dd >> 16));
      int sc_lo, m_lo, sc_hi, m_hi;
      ScaleMinK4(2 * p, block[1], block[2], block[3], &sc_lo, &m_lo);
      ScaleMinK4(2 * p + 1, block[1], block[2], block[3], &sc_hi, &m_hi);
      const float d1 = __fmul_rn(d, static_cast<float>(sc_lo)), m1 = __fmul_rn(dmin, static_cast<float>(m_lo));
      const float d2 = __fmul_rn(d, static_cast<float>(sc_hi)), m2 = __fmul_rn(dmin, static_cast<float>(m_hi));
      const uint32_t q = block[4 + word];
      float* out = a.h + b * kSuperBlock + 64 * p + 4 * c;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[i] = __fsub_rn(__fmul_rn(d1, static_cast<float>((q >> (8 * i)) & 0xF)), m1);
        out[32 + i] = __fsub_rn(__fmul_rn(d2, static_cast<float>((q >> (8 * i + 4)) & 0xF)), m2);
      }
    }
  } else if (a.type == GUFO_CUDA_Q6_K) {
    for (int item = threadIdx.x; item < blocks * 64; item += kSmallThreads) {
      const int b = item >> 6, half = (item >> 5) & 1, l = item & 31;
      const Q6KBlock block = Q6KBlockAt(row, blocks, b);
      const uint8_t* ql = block.ql + 64 * half;
      const uint8_t* qh = block.qh + 32 * half;
      const int8_t* sc = block.sc + 8 * half + (l >> 4);
      const float d = HalfBitsToFloat(*reinterpret_cast<const uint16_t*>(block.d));
      const int x = ql[l], c = ql[l + 32], h = qh[l];
      float* out = a.h + b * kSuperBlock + 128 * half + l;
      out[0] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[0])), static_cast<float>(((x & 0xF) | ((h & 3) << 4)) - 32));
      out[32] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[2])), static_cast<float>(((c & 0xF) | (((h >> 2) & 3) << 4)) - 32));
      out[64] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[4])), static_cast<float>(((x >> 4) | (((h >> 4) & 3) << 4)) - 32));
      out[96] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[6])), static_cast<float>(((c >> 4) | (((h >> 6) & 3) << 4)) - 32));
    }
  } else {
    for (int i = threadIdx.x; i < a.cols; i += kSmallThreads) {
      a.h[i] = reinterpret_cast<const float*>(row)[i];
    }
  }
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

struct AttnArgs {
  int heads, kv_heads, head_dim, rope_dim, max_positions;
  float rms_eps;
  const int* position;
  const float* in;          // [q and gate (2 heads hd, per head q | gate) | k | v]
  const float* q_norm;
  const float* k_norm;
  const float* inv_freq;    // [rope_dim / 2]
  __half* keys;             // [max_positions][kv_heads * hd]
  __half* values;
  float* queries;           // [heads][hd]
  float* partials;          // [kv_heads][splits][group][hd + 2]
  float* ctx;               // [heads][hd]
  int offset = 0;           // the token sits at *position + offset
};

// q/k RMSNorm and RoPE; appends k and v to the cache in fp16
// (decoder.cpp:280-323). Block h < heads: query head h; then one per KV head.
__global__ void __launch_bounds__(kSmallThreads)
AttnPrepKernel(const __grid_constant__ AttnArgs a) {
  __shared__ float scratch[kSmallThreads / 32];
  __shared__ float vec[kMaxPerLane * 32];
  GridLaunchDependents();
  GridDependencyWait();
  const int hd = a.head_dim;
  const int half = a.rope_dim / 2;
  const int pos = *a.position + a.offset;
  const int head = blockIdx.x;
  const bool is_query = head < a.heads;
  const int kh = head - a.heads;
  const float* x = is_query ? a.in + static_cast<size_t>(head) * 2 * hd
                            : a.in + static_cast<size_t>(a.heads) * 2 * hd + kh * hd;
  const float* w = is_query ? a.q_norm : a.k_norm;
  const int e = threadIdx.x;
  const float v = e < hd ? x[e] : 0.f;
  const float total = BlockSum256(v * v, scratch);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(hd) + a.rms_eps);
  if (e < hd) {
    vec[e] = v * inv * w[e];
  }
  __syncthreads();
  float out = e < hd ? vec[e] : 0.f;
  if (e < 2 * half) {
    const int i = e < half ? e : e - half;
    const double angle = static_cast<double>(pos) * static_cast<double>(a.inv_freq[i]);
    const float cs = static_cast<float>(cos(angle));
    const float sn = static_cast<float>(sin(angle));
    const float lo = vec[i], hi = vec[i + half];
    out = e < half ? lo * cs - hi * sn : lo * sn + hi * cs;
  }
  if (e < hd) {
    if (is_query) {
      a.queries[head * hd + e] = out;
    } else {
      const size_t at = (static_cast<size_t>(pos) * a.kv_heads + kh) * hd + e;
      a.keys[at] = __float2half_rn(out);
      const float val = a.in[static_cast<size_t>(a.heads) * 2 * hd + a.kv_heads * hd + kh * hd + e];
      a.values[at] = __float2half_rn(val);
    }
  }
}

// One slice of the cached positions for one KV head and the query heads that
// share it: partial softmax (weighted values, max, sum) per query head
// (the split-K jobs of decoder.cpp:326-381). grid = (splits, kv_heads).
__global__ void __launch_bounds__(kSmallThreads)
AttnSliceKernel(const __grid_constant__ AttnArgs a) {
  __shared__ float q_sh[kMaxGroup][kMaxPerLane * 32];
  __shared__ float merge_m[kSmallThreads / 32][kMaxGroup];
  __shared__ float merge_l[kSmallThreads / 32][kMaxGroup];
  __shared__ float merge_acc[kSmallThreads / 32][kMaxPerLane * 32];
  GridLaunchDependents();
  GridDependencyWait();
  const int hd = a.head_dim;
  const int per = hd / 32;
  const int group = a.heads / a.kv_heads;
  const int kh = blockIdx.y;
  const int length = *a.position + a.offset + 1;
  const int slice = (length + kAttnSplits - 1) / kAttnSplits;
  const int begin = blockIdx.x * slice;
  const int end = min(length, begin + slice);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float scale = 1.0f / sqrtf(static_cast<float>(hd));
  for (int i = threadIdx.x; i < group * hd; i += kSmallThreads) {
    q_sh[i / hd][i % hd] = a.queries[(kh * group) * hd + i];
  }
  __syncthreads();
  float m[kMaxGroup], l[kMaxGroup], acc[kMaxGroup][kMaxPerLane];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      acc[g][i] = 0.f;
    }
  }
  const int kv = a.kv_heads * hd;
  for (int j = begin + warp; j < end; j += kSmallThreads / 32) {
    const __half* key = a.keys + static_cast<size_t>(j) * kv + kh * hd + lane * per;
    const __half* val = a.values + static_cast<size_t>(j) * kv + kh * hd + lane * per;
    float kf[kMaxPerLane], vf[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      kf[i] = i < per ? __half2float(key[i]) : 0.f;
      vf[i] = i < per ? __half2float(val[i]) : 0.f;
    }
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
      if (g < group) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
          if (i < per) {
            dot = fmaf(q_sh[g][lane * per + i], kf[i], dot);
          }
        }
        const float s = WarpSum(dot) * scale;
        const float m_new = fmaxf(m[g], s);
        const float keep = expf(m[g] - m_new);   // 0 on the first position
        const float p = expf(s - m_new);
        l[g] = l[g] * keep + p;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
          acc[g][i] = acc[g][i] * keep + p * vf[i];
        }
        m[g] = m_new;
      }
    }
  }
  // Merge the warps, one query head at a time.
  for (int g = 0; g < group; ++g) {
    float mg = -INFINITY, lg = 0.f, ag[kMaxPerLane];
#pragma unroll
    for (int gg = 0; gg < kMaxGroup; ++gg) {
      if (gg == g) {
        mg = m[gg];
        lg = l[gg];
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
          ag[i] = acc[gg][i];
        }
      }
    }
    __syncthreads();
    if (lane == 0) {
      merge_m[warp][0] = mg;
    }
    __syncthreads();
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kSmallThreads / 32; ++w) {
      top = fmaxf(top, merge_m[w][0]);
    }
    const float wgt = mg == -INFINITY ? 0.f : expf(mg - top);
    if (lane == 0) {
      merge_l[warp][0] = lg * wgt;
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      if (i < per) {
        merge_acc[warp][lane * per + i] = ag[i] * wgt;
      }
    }
    __syncthreads();
    float* out = a.partials + ((static_cast<size_t>(kh) * kAttnSplits + blockIdx.x) * group + g) * (hd + 2);
    for (int e = threadIdx.x; e < hd; e += kSmallThreads) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kSmallThreads / 32; ++w) {
        total += merge_acc[w][e];
      }
      out[e] = total;
    }
    if (threadIdx.x == 0) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kSmallThreads / 32; ++w) {
        total += merge_l[w][0];
      }
      out[hd] = top;
      out[hd + 1] = total;
    }
  }
}

// Merges the slices per query head and applies the output gate
// (decoder.cpp:383-411). grid = heads.
__global__ void __launch_bounds__(kSmallThreads)
AttnMergeKernel(const __grid_constant__ AttnArgs a) {
  GridLaunchDependents();
  GridDependencyWait();
  const int hd = a.head_dim;
  const int group = a.heads / a.kv_heads;
  const int qh = blockIdx.x;
  const int kh = qh / group, g = qh % group;
  auto slice = [&](int s) {
    return a.partials + ((static_cast<size_t>(kh) * kAttnSplits + s) * group + g) * (hd + 2);
  };
  float top = -INFINITY;
  for (int s = 0; s < kAttnSplits; ++s) {
    top = fmaxf(top, slice(s)[hd]);
  }
  float total = 0.f;
  float wgt[kAttnSplits];
  for (int s = 0; s < kAttnSplits; ++s) {
    const float ms = slice(s)[hd];
    wgt[s] = ms == -INFINITY ? 0.f : expf(ms - top);
    total += wgt[s] * slice(s)[hd + 1];
  }
  const float inv_total = 1.0f / total;
  const float* gate = a.in + static_cast<size_t>(qh) * 2 * hd + hd;
  for (int e = threadIdx.x; e < hd; e += kSmallThreads) {
    float out = 0.f;
    for (int s = 0; s < kAttnSplits; ++s) {
      out += wgt[s] * slice(s)[e];
    }
    a.ctx[qh * hd + e] = out * (inv_total * SigmoidF(gate[e]));
  }
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
  cudaGraphExec_t graph[2][2][2] = {};
  int64_t graph_kernels[2][2][2] = {};
  int eager_runs[2][2] = {};
  std::vector<void*> owned;   // every device allocation, for destroy

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
  const float* norm_w = nullptr;
  float* h_out = nullptr;
  int* advance = nullptr;
};

// One stage's product for `tokens` rows with its input fused into the GEMV
// kernels where every part allows it; otherwise the input is materialised by the
// small kernels first. `scratch` holds the materialised / normed rows.
int FusedProduct(gufo_cuda_ctx* ctx, float rms_eps, const GemvArgs& stage, const Input& in, float* scratch,
                 float* y, int tokens) {
  const dim3 block(kSmallThreads);
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
                 int tokens) {
  return FusedProduct(d->ctx, d->c.rms_eps, stage, in, scratch, y, tokens);
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
int EnqueueStep(gufo_cuda_decoder* d, int parity, bool want_logits, int tokens) {
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
    GUFO_STEP_TRY(FusedProduct(d, l.ffn_in, norm2, d->normed, d->ffn, tokens));
    Mark(d, GUFO_CUDA_TIMELINE_FFN_IN);
    cur ^= 1;
    Input swiglu{kPrologueSwiGlu};
    swiglu.x = d->ffn;
    GUFO_STEP_TRY(FusedProduct(d, l.ffn_down, swiglu, d->act, d->out, tokens));
    if (c.experts > 0) {
      // Decoder::MoeFfn (decoder.cpp:535-557): d->out holds the shared
      // expert's output, d->normed the layer's normed input.
      GemvArgs router = l.router;
      router.x = d->normed;
      router.y = d->router;
      GUFO_STEP_TRY(LaunchGemv(ctx, router, tokens));
      GUFO_STEP_TRY(EnqueueRoute(ctx, d->router, c.experts + 1, tokens, c.experts, c.experts_used, d->chosen,
                                 d->route_weights, d->shared_scale));
      GUFO_STEP_TRY(EnqueueExpertFfn(ctx, l.bank, d->chosen, tokens * c.experts_used, d->normed, c.hidden,
                                     c.experts_used, d->expert_ffn, d->expert_act, d->expert_out));
      GUFO_STEP_TRY(EnqueueMoeCombine(ctx, d->out, d->shared_scale, d->route_weights, d->expert_out, tokens,
                                      c.experts_used, c.hidden, d->out));
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
  if (want_logits) {
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
  return gufo::FusedProduct(ctx, in->rms_eps, stage, input, in->scratch, y, tokens);
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
              {&d->in, two * in_max}, {&d->mixed, two * mixed}, {&d->out, two * c.hidden},
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
  const int pair = count - 1, with = want_logits != 0 ? 1 : 0;
  auto enqueue = [&]() { return gufo::EnqueueStep(d, parity, with != 0, count); };
  if (d->c.use_graph && d->eager_runs[pair][with] >= 2 && !d->timeline) {
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
    ++d->eager_runs[pair][with];
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
  if (host_logits != nullptr) {
    GUFO_CUDA_TRY(cudaMemcpyAsync(host_logits, d->logits, static_cast<size_t>(count) * d->c.vocab * 4,
                                  cudaMemcpyDeviceToHost, ctx->stream));
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
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
