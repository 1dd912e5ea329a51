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

namespace {

// The grouped product of narrow Q4_K matrices (1, 2 or 4 blocks of 256 values a
// row: an expert's down projection, 2048 x 512 here) with one fp32 input per
// group. The 16-row x 8-block tiles of the fast GEMV leave six of eight warps
// idle on such rows and pay an input conversion per tile; here sixteen lanes
// take a block of a row (a lane: eight bytes of codes, i.e. eight values each of
// the sub-blocks 2c and 2c + 1, with the sixteen inputs they meet held in
// registers for all of the warp's rows), dequantize as the reference does
// (w = d * sc * q - dmin * m, DequantQ4_K, src/core/quant.cpp:64-96) and reduce
// over the row's lanes. `x` is plain, or [gate | up] per group when `swiglu`.
struct NarrowArgs {
  const uint8_t* w;      // experts stacked along the rows
  int rows;              // of one expert
  int row_bytes;
  const int* ids;        // [groups], < 0: nothing to do
  const float* x;
  int x_stride;          // floats between the groups' inputs
  int x_div;             // groups per input
  int swiglu;
  float* y;
  int y_stride;          // floats between the groups' outputs
};

constexpr int kNarrowPasses = 8;   // rows (or row pairs) a warp multiplies, loads issued together

__device__ __forceinline__ float NarrowSilu(float v) { return v * (1.0f / (1.0f + expf(-v))); }

template <int BLOCKS>
__global__ void __launch_bounds__(256)
NarrowGroupedQ4K(const __grid_constant__ NarrowArgs a) {
  constexpr int kSlots = 16 * BLOCKS;                       // lane slots a row
  constexpr int kPer = kSlots > 32 ? kSlots / 32 : 1;       // slots a lane
  constexpr int kRowsAtOnce = kSlots < 32 ? 32 / kSlots : 1;
  constexpr int kWarpRows = kNarrowPasses * kRowsAtOnce;
  GridLaunchDependents();
  GridDependencyWait();   // the ids and the inputs come from earlier kernels
  const int group = blockIdx.y;
  const int id = a.ids[group];
  if (id < 0) {
    return;
  }
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int first = (blockIdx.x * 8 + warp) * kWarpRows;
  const uint8_t* matrix = a.w + static_cast<size_t>(id) * a.rows * a.row_bytes;
  const float* x = a.x + static_cast<size_t>(group / (a.x_div > 1 ? a.x_div : 1)) * a.x_stride;
  const int cols = 256 * BLOCKS;
  // This lane's slots: block b, 32-byte chunk c of its codes, eight-byte part p.
  int at[kPer];       // byte offset of the block in the row
  int part[kPer];     // offset of the eight code bytes behind the block's 16-byte head
  int pair[kPer];     // c: sub-blocks 2c (low nibbles) and 2c + 1 (high)
  float lo[kPer][8], hi[kPer][8], lo_sum[kPer], hi_sum[kPer];
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int slot = (lane + 32 * j) % kSlots;
    const int b = slot >> 4;
    const int c = (slot >> 2) & 3;
    const int p = slot & 3;
    at[j] = b * kQ4KBytes;
    part[j] = 32 * c + 8 * p;
    pair[j] = c;
    const int col = 256 * b + 64 * c + 8 * p;
    lo_sum[j] = hi_sum[j] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (a.swiglu) {
        lo[j][i] = NarrowSilu(x[col + i]) * x[cols + col + i];
        hi[j][i] = NarrowSilu(x[col + 32 + i]) * x[cols + col + 32 + i];
      } else {
        lo[j][i] = x[col + i];
        hi[j][i] = x[col + 32 + i];
      }
      lo_sum[j] += lo[j][i];
      hi_sum[j] += hi[j][i];
    }
  }
  const int sub = kRowsAtOnce > 1 ? lane / kSlots : 0;   // which of the rows taken at once
  uint4 head[kNarrowPasses][kPer];
  uint2 codes[kNarrowPasses][kPer];
#pragma unroll
  for (int r = 0; r < kNarrowPasses; ++r) {
    // Rows past the end repeat the last row; their sums are not stored.
    const int row = min(first + r * kRowsAtOnce + sub, a.rows - 1);
    const uint8_t* from = matrix + static_cast<size_t>(row) * a.row_bytes;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      head[r][j] = *reinterpret_cast<const uint4*>(from + at[j]);
      codes[r][j] = *reinterpret_cast<const uint2*>(from + at[j] + 16 + part[j]);
    }
  }
#pragma unroll
  for (int r = 0; r < kNarrowPasses; ++r) {
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const float d = HalfBitsToFloat(static_cast<uint16_t>(head[r][j].x & 0xFFFF));
      const float dmin = HalfBitsToFloat(static_cast<uint16_t>(head[r][j].x >> 16));
      int sc_lo, m_lo, sc_hi, m_hi;
      ScaleMinK4(2 * pair[j], head[r][j].y, head[r][j].z, head[r][j].w, &sc_lo, &m_lo);
      ScaleMinK4(2 * pair[j] + 1, head[r][j].y, head[r][j].z, head[r][j].w, &sc_hi, &m_hi);
      float dot_lo = 0.f, dot_hi = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t word = i < 4 ? codes[r][j].x : codes[r][j].y;
        const uint32_t byte = (word >> (8 * (i & 3))) & 0xFFu;
        dot_lo = fmaf(static_cast<float>(byte & 15u), lo[j][i], dot_lo);
        dot_hi = fmaf(static_cast<float>(byte >> 4), hi[j][i], dot_hi);
      }
      sum += d * (static_cast<float>(sc_lo) * dot_lo + static_cast<float>(sc_hi) * dot_hi) -
             dmin * (static_cast<float>(m_lo) * lo_sum[j] + static_cast<float>(m_hi) * hi_sum[j]);
    }
#pragma unroll
    for (int o = kSlots < 32 ? kSlots / 2 : 16; o > 0; o >>= 1) {
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    }
    const int row = first + r * kRowsAtOnce + sub;
    if ((lane % (kSlots < 32 ? kSlots : 32)) == 0 && row < a.rows) {
      a.y[static_cast<size_t>(group) * a.y_stride + row] = sum;
    }
  }
}

template <int BLOCKS>
int LaunchNarrow(gufo_cuda_ctx* ctx, const NarrowArgs& args, int groups) {
  constexpr int kSlots = 16 * BLOCKS;
  constexpr int kBlockRows = 8 * kNarrowPasses * (kSlots < 32 ? 32 / kSlots : 1);
  GUFO_CUDA_TRY(LaunchOverlapped(NarrowGroupedQ4K<BLOCKS>, dim3((args.rows + kBlockRows - 1) / kBlockRows, groups),
                                 dim3(256), 0, ctx->stream, 1, args));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

// Whether the narrow kernel takes a grouped product of one Q4_K part.
bool NarrowFits(const GemvArgs& g) {
  const int blocks = g.cols / kSuperBlock;
  return g.nparts == 1 && g.parts[0].type == GUFO_CUDA_Q4_K && g.cols % kSuperBlock == 0 &&
         (blocks == 1 || blocks == 2 || blocks == 4);
}

int LaunchNarrowGrouped(gufo_cuda_ctx* ctx, const GemvArgs& g, bool swiglu) {
  NarrowArgs args{};
  args.w = g.parts[0].data;
  args.rows = g.parts[0].rows;
  args.row_bytes = g.parts[0].row_bytes;
  args.ids = g.group_ids;
  args.x = g.x;
  args.x_stride = g.x_group_stride;
  args.x_div = g.x_group_div;
  args.swiglu = swiglu ? 1 : 0;
  args.y = g.y + g.parts[0].out_offset;
  args.y_stride = g.y_group_stride;
  switch (g.cols / kSuperBlock) {
    case 1: return LaunchNarrow<1>(ctx, args, g.groups);
    case 2: return LaunchNarrow<2>(ctx, args, g.groups);
    default: return LaunchNarrow<4>(ctx, args, g.groups);
  }
}

// The down product of a token's k (<= 8) chosen experts and Decoder::MoeFfn's
// weighted sum in one launch (decoder.cpp:541-556): out[t][row] = shared[t][row] *
// scale[t] + the sum, in slot order, of weights[t][s] * (row of expert ids[t][s]
// times act[t][s]). A warp takes a row (BLOCKS = 1: two rows) of all k experts at
// once: k row loads in flight, the k activated inputs of the token in shared
// memory. A slot with ids < 0 adds nothing.
struct NarrowCombineArgs {
  const uint8_t* w;
  int rows;
  int row_bytes;
  const int* ids;          // [tokens][k]
  const float* weights;    // [tokens][k]
  const float* scale;      // [tokens]
  const float* shared;     // [tokens][rows]
  const float* act;        // [tokens][k][256 * BLOCKS]
  int k;
  float* out;              // [tokens][rows]; may be shared
};

constexpr int kCombineSlots = 8;

template <int BLOCKS>
__global__ void __launch_bounds__(256)
NarrowCombineQ4K(const __grid_constant__ NarrowCombineArgs a) {
  constexpr int kSlots = 16 * BLOCKS;
  constexpr int kPer = kSlots > 32 ? kSlots / 32 : 1;
  constexpr int kRowsAtOnce = kSlots < 32 ? 32 / kSlots : 1;
  constexpr int kCols = 256 * BLOCKS;
  __shared__ __align__(16) float xs[kCombineSlots][kCols];
  GridLaunchDependents();
  GridDependencyWait();
  const int token = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = kRowsAtOnce > 1 ? lane / kSlots : 0;
  const int row = (blockIdx.x * 8 + warp) * kRowsAtOnce + sub;
  const int load_row = min(row, a.rows - 1);
  int at[kPer], part[kPer], pair[kPer], col[kPer];
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int slot = (lane + 32 * j) % kSlots;
    const int b = slot >> 4;
    const int c = (slot >> 2) & 3;
    const int p = slot & 3;
    at[j] = b * kQ4KBytes;
    part[j] = 32 * c + 8 * p;
    pair[j] = c;
    col[j] = 256 * b + 64 * c + 8 * p;
  }
  // The k rows first (they come from HBM), then the inputs.
  uint4 head[kCombineSlots][kPer];
  uint2 codes[kCombineSlots][kPer];
  int id[kCombineSlots];
#pragma unroll
  for (int s = 0; s < kCombineSlots; ++s) {
    id[s] = s < a.k ? a.ids[token * a.k + s] : -1;
    if (id[s] >= 0) {
      const uint8_t* from = a.w + (static_cast<size_t>(id[s]) * a.rows + load_row) * a.row_bytes;
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        head[s][j] = *reinterpret_cast<const uint4*>(from + at[j]);
        codes[s][j] = *reinterpret_cast<const uint2*>(from + at[j] + 16 + part[j]);
      }
    }
  }
  for (int i = threadIdx.x * 4; i < a.k * kCols; i += 256 * 4) {
    const int s = i / kCols;
    *reinterpret_cast<float4*>(&xs[s][i - s * kCols]) =
        *reinterpret_cast<const float4*>(a.act + (static_cast<size_t>(token) * a.k + s) * kCols + (i - s * kCols));
  }
  __syncthreads();
  float sum[kCombineSlots];
#pragma unroll
  for (int s = 0; s < kCombineSlots; ++s) {
    sum[s] = 0.f;
    if (id[s] >= 0) {
#pragma unroll
      for (int j = 0; j < kPer; ++j) {
        const float4 l0 = *reinterpret_cast<const float4*>(&xs[s][col[j]]);
        const float4 l1 = *reinterpret_cast<const float4*>(&xs[s][col[j] + 4]);
        const float4 h0 = *reinterpret_cast<const float4*>(&xs[s][col[j] + 32]);
        const float4 h1 = *reinterpret_cast<const float4*>(&xs[s][col[j] + 36]);
        const float lo[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
        const float hi[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
        const float d = HalfBitsToFloat(static_cast<uint16_t>(head[s][j].x & 0xFFFF));
        const float dmin = HalfBitsToFloat(static_cast<uint16_t>(head[s][j].x >> 16));
        int sc_lo, m_lo, sc_hi, m_hi;
        ScaleMinK4(2 * pair[j], head[s][j].y, head[s][j].z, head[s][j].w, &sc_lo, &m_lo);
        ScaleMinK4(2 * pair[j] + 1, head[s][j].y, head[s][j].z, head[s][j].w, &sc_hi, &m_hi);
        float dot_lo = 0.f, dot_hi = 0.f, lo_sum = 0.f, hi_sum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t word = i < 4 ? codes[s][j].x : codes[s][j].y;
          const uint32_t byte = (word >> (8 * (i & 3))) & 0xFFu;
          dot_lo = fmaf(static_cast<float>(byte & 15u), lo[i], dot_lo);
          dot_hi = fmaf(static_cast<float>(byte >> 4), hi[i], dot_hi);
          lo_sum += lo[i];
          hi_sum += hi[i];
        }
        sum[s] += d * (static_cast<float>(sc_lo) * dot_lo + static_cast<float>(sc_hi) * dot_hi) -
                  dmin * (static_cast<float>(m_lo) * lo_sum + static_cast<float>(m_hi) * hi_sum);
      }
    }
  }
#pragma unroll
  for (int o = kSlots < 32 ? kSlots / 2 : 16; o > 0; o >>= 1) {
#pragma unroll
    for (int s = 0; s < kCombineSlots; ++s) {
      sum[s] += __shfl_xor_sync(0xFFFFFFFFu, sum[s], o);
    }
  }
  if ((lane % (kSlots < 32 ? kSlots : 32)) == 0 && row < a.rows) {
    const size_t at_out = static_cast<size_t>(token) * a.rows + row;
    float v = a.shared[at_out] * a.scale[token];
#pragma unroll
    for (int s = 0; s < kCombineSlots; ++s) {
      if (s < a.k && id[s] >= 0) {
        v = fmaf(a.weights[token * a.k + s], sum[s], v);
      }
    }
    a.out[at_out] = v;
  }
}

template <int BLOCKS>
int LaunchNarrowCombine(gufo_cuda_ctx* ctx, const NarrowCombineArgs& args, int tokens) {
  constexpr int kBlockRows = 8 * (16 * BLOCKS < 32 ? 32 / (16 * BLOCKS) : 1);
  GUFO_CUDA_TRY(LaunchOverlapped(NarrowCombineQ4K<BLOCKS>, dim3((args.rows + kBlockRows - 1) / kBlockRows, tokens),
                                 dim3(256), 0, ctx->stream, 1, args));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

}  // namespace

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
    return NarrowFits(down) ? LaunchNarrowGrouped(ctx, down, false)
                            : LaunchGemvGrouped(ctx, down, kProloguePlain, nullptr);
  }
  int rc = LaunchGemvGrouped(ctx, in, kProloguePlain, nullptr);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  down.x = ffn;
  down.x_group_stride = 2 * bank.expert_ffn;
  return NarrowFits(down) ? LaunchNarrowGrouped(ctx, down, true)
                          : LaunchGemvGrouped(ctx, down, kPrologueSwiGlu, act);
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

int EnqueueMoeFfn(gufo_cuda_ctx* ctx, const ExpertBank& bank, const int* ids, const float* weights,
                  const float* scale, int tokens, int k, const float* x, int x_stride, const float* shared,
                  float* ffn, float* act, float* expert_out, float* out) {
  if (tokens <= 0 || k <= 0 || ids == nullptr || weights == nullptr || scale == nullptr || x == nullptr ||
      shared == nullptr || ffn == nullptr || act == nullptr || expert_out == nullptr || out == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "moe ffn: null pointer or no tokens");
  }
  GemvArgs in = bank.in;
  in.x = x;
  in.y = act;
  in.group_ids = ids;
  in.groups = tokens * k;
  in.x_group_stride = x_stride;
  in.x_group_div = k;
  in.y_group_stride = bank.expert_ffn;
  GemvArgs down = bank.down;
  const int blocks = down.cols / kSuperBlock;
  if (k <= kCombineSlots && NarrowFits(down) && blocks <= 2 && GroupedSwiGluInProduct(ctx, in)) {
    // Two launches: gate / up with the SwiGLU in its epilogue, then the down rows
    // of a token's experts with the weighted sum.
    const int rc = LaunchGemvGrouped(ctx, in, kProloguePlain, nullptr, true);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
    NarrowCombineArgs args{};
    args.w = down.parts[0].data;
    args.rows = down.parts[0].rows;
    args.row_bytes = down.parts[0].row_bytes;
    args.ids = ids;
    args.weights = weights;
    args.scale = scale;
    args.shared = shared;
    args.act = act;
    args.k = k;
    args.out = out;
    return blocks == 1 ? LaunchNarrowCombine<1>(ctx, args, tokens) : LaunchNarrowCombine<2>(ctx, args, tokens);
  }
  const int rc = EnqueueExpertFfn(ctx, bank, ids, tokens * k, x, x_stride, k, ffn, act, expert_out);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  return EnqueueMoeCombine(ctx, shared, scale, weights, expert_out, tokens, k, bank.hidden, out);
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

int gufo_cuda_moe_ffn_device(gufo_cuda_ctx* ctx, const gufo_cuda_expert_bank* bank, const int* ids,
                             const float* weights, const float* scale, int tokens, int k, const float* x,
                             int64_t x_stride, const float* shared, float* ffn, float* act, float* expert_out,
                             float* out) {
  if (ctx == nullptr || bank == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "moe ffn: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::ExpertBank built;
  const int rc = gufo::BuildExpertBank(ctx, *bank, &built);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  if (x_stride != 0 && x_stride < bank->hidden) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "moe ffn: x_stride is 0 (shared input) or at least hidden");
  }
  return gufo::EnqueueMoeFfn(ctx, built, ids, weights, scale, tokens, k, x, static_cast<int>(x_stride), shared, ffn,
                             act, expert_out, out);
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
