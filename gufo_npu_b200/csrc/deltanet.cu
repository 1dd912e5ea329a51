// The Gated DeltaNet decode step (Mixer::Linear,
// src/models/qwen35/decoder.cpp:161-265 in the reference; its delta rule,
// lines 234-257, restated blockwise in src/models/qwen35_2b/deltanet.cpp:56-82).
//
// Per value head the fp32 state S[i (key)][j (value)] is read from HBM once,
// kept on chip across the retrieval pass (u = (decay S)^T k), the rank-1 update
// (S' = decay S + k delta^T) and the readout (y = S'^T q), and written once:
// algorithmic traffic is 2 * dk * dk * 4 bytes per head, the HBM roofline of
// this kernel. Columns of S evolve independently
// (src/models/qwen35/prefill_mixer.cpp:662-667), so one thread block takes one
// (sequence, value head) and each of its warps one tile of 32 columns.
//
// Warp layout: lane = 8 * ig + jq; jq owns four adjacent columns (one float4),
// ig owns rows ig, ig + 4, ..., so one load instruction of a warp covers four
// 128-byte row segments. A lane keeps its dk / 4 float4 of S (128 registers at
// dk = 128) from the loads to the stores: all of a tile's state is requested
// from HBM at once, the column sums of the two passes need only two shuffle
// steps, and the block meets just once, for the gated RMSNorm over the head's
// dk outputs.
#include "common.cuh"

#include <vector>

namespace gufo {

constexpr int kMaxHeadDim = 128;
constexpr int kDeltaThreads = kMaxHeadDim;            // one thread per column
constexpr int kMaxSeqs = 16;                          // descriptors per launch

struct DeltaRuleArgs {
  gufo_cuda_delta_seq seq[kMaxSeqs];
  int key_heads;
  int value_heads;
  int head_dim;
  int early_state;   // as in LinearArgs below
};

struct LinearArgs {
  gufo_cuda_linear_seq seq[kMaxSeqs];
  int key_heads;
  int value_heads;
  int head_dim;
  int conv_kernel;
  float rms_eps;
  const float* conv;
  const float* ssm_a;
  const float* dt_bias;
  const float* ssm_norm;
  // When the caller knows that no kernel shortly before this one in the stream
  // wrote the states, their loads may start ahead of the dependency wait.
  int early_state;
  // Non-null alpha_w: the gates come from these rows instead of the input row.
  DeltaNetGateRows gate_rows;
  const float* gate_x[kMaxSeqs];   // per sequence, or null for gate_rows.x
};

namespace {

struct DeltaShared {
  float q[kMaxHeadDim];
  float k[kMaxHeadDim];
  float v[kMaxHeadDim];
  float y[kMaxHeadDim];
  float gate[2];                              // decay, beta
  float scratch[5 * (2 * kDeltaThreads / 32)];   // up to five sums a warp (BlockSum5)
};

// A warp's tile of COLS (8 or 16) adjacent columns of a head's state: a lane
// holds rows ig, ig + 32 / G, ... (ig = lane / G, G = COLS / 4) of four adjacent
// columns (4 * (lane % G)). Narrow tiles mean many warps per head.
template <int COLS>
struct NarrowTile {
  static constexpr int kGroups = COLS / 4;                 // lanes across the columns
  static constexpr int kRowGroups = 32 / kGroups;
  static constexpr int kRowsPerLane = kMaxHeadDim / kRowGroups;
  float4 s[kRowsPerLane];
};

template <int COLS>
__device__ __forceinline__ void LoadNarrowTile(NarrowTile<COLS>& tile, const float* __restrict__ src, int dk,
                                               int tile_index) {
  using T = NarrowTile<COLS>;
  const int lane = threadIdx.x & 31;
  const int col = tile_index * COLS + 4 * (lane % T::kGroups);
  const int ig = lane / T::kGroups;
  const int rows = dk / T::kRowGroups;
#pragma unroll
  for (int r = 0; r < T::kRowsPerLane; ++r) {
    if (r < rows) {
      tile.s[r] = *reinterpret_cast<const float4*>(src + static_cast<size_t>(r * T::kRowGroups + ig) * dk + col);
    }
  }
}

// Sum over the warp's row groups; every lane gets its columns' totals.
template <int COLS>
__device__ __forceinline__ float4 NarrowColumnSum(float4 v) {
#pragma unroll
  for (int o = NarrowTile<COLS>::kGroups; o <= 16; o <<= 1) {
    v.x += __shfl_xor_sync(0xFFFFFFFFu, v.x, o);
    v.y += __shfl_xor_sync(0xFFFFFFFFu, v.y, o);
    v.z += __shfl_xor_sync(0xFFFFFFFFu, v.z, o);
    v.w += __shfl_xor_sync(0xFFFFFFFFu, v.w, o);
  }
  return v;
}

// The delta rule on this warp's column tile. sh.q, sh.k, sh.v and sh.gate are
// ready. Writes S' to dst and the tile's outputs to sh.y (no barrier); with
// `squares`, lane 0 also leaves the sum of the squares of the tile's outputs there.
template <int COLS>
__device__ __forceinline__ void NarrowDeltaTile(NarrowTile<COLS>& tile, float* __restrict__ dst, int dk,
                                                int tile_index, DeltaShared& sh, float* squares = nullptr) {
  using T = NarrowTile<COLS>;
  const int lane = threadIdx.x & 31;
  const int col = tile_index * COLS + 4 * (lane % T::kGroups);
  const int ig = lane / T::kGroups;
  const int rows = dk / T::kRowGroups;
  const float decay = sh.gate[0];
  const float beta = sh.gate[1];
  float4 (&s)[T::kRowsPerLane] = tile.s;
  // Pass 1: u_j = sum_i S_ij * (k_i * decay).
  float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < T::kRowsPerLane; ++r) {
    if (r < rows) {
      const float ki = sh.k[r * T::kRowGroups + ig] * decay;
      u.x = fmaf(s[r].x, ki, u.x);
      u.y = fmaf(s[r].y, ki, u.y);
      u.z = fmaf(s[r].z, ki, u.z);
      u.w = fmaf(s[r].w, ki, u.w);
    }
  }
  u = NarrowColumnSum<COLS>(u);
  const float4 v = *reinterpret_cast<const float4*>(&sh.v[col]);
  float4 delta;
  delta.x = beta * (v.x - u.x);
  delta.y = beta * (v.y - u.y);
  delta.z = beta * (v.z - u.z);
  delta.w = beta * (v.w - u.w);
  // Pass 2: S'_ij = S_ij * decay + k_i * delta_j; y_j = sum_i S'_ij * q_i.
  float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < T::kRowsPerLane; ++r) {
    if (r < rows) {
      const int i = r * T::kRowGroups + ig;
      const float ki = sh.k[i];
      const float qi = sh.q[i];
      float4 n;
      n.x = fmaf(s[r].x, decay, ki * delta.x);
      n.y = fmaf(s[r].y, decay, ki * delta.y);
      n.z = fmaf(s[r].z, decay, ki * delta.z);
      n.w = fmaf(s[r].w, decay, ki * delta.w);
      *reinterpret_cast<float4*>(dst + static_cast<size_t>(i) * dk + col) = n;
      y.x = fmaf(n.x, qi, y.x);
      y.y = fmaf(n.y, qi, y.y);
      y.z = fmaf(n.z, qi, y.z);
      y.w = fmaf(n.w, qi, y.w);
    }
  }
  y = NarrowColumnSum<COLS>(y);
  if (ig == 0) {
    *reinterpret_cast<float4*>(&sh.y[col]) = y;
  }
  if (squares != nullptr) {
    // Lanes 0 .. kGroups - 1 hold the tile's COLS outputs.
    float sq = ig == 0 ? y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w : 0.f;
#pragma unroll
    for (int o = T::kGroups / 2; o > 0; o >>= 1) {
      sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
    }
    if (lane == 0) {
      *squares = sq;
    }
  }
}

constexpr int kStepCols = 16;   // columns per warp in the decode step's kernel
constexpr int kRuleCols = 16;   // and in the stand-alone delta rule (8: 4.9 us for config 3, 16: 4.1, 32: 4.6)

// Gates given: one warp per thread block, grid = (dk / 16, value_heads,
// sequences). The tiles of a head need nothing from one another here, and
// many small blocks per SM let one tile's stores overlap another's loads
// (16-column tiles: 1024 warps for eight sequences of sixteen heads).
__global__ void __launch_bounds__(32)
DeltaRuleKernel(const __grid_constant__ DeltaRuleArgs args) {
  __shared__ __align__(16) DeltaShared sh;
  const gufo_cuda_delta_seq& seq = args.seq[blockIdx.z];
  const int head = blockIdx.y;
  const int tile = blockIdx.x;
  const int dk = args.head_dim;
  const int kh = head % args.key_heads;
  const int lane = threadIdx.x;
  const size_t state_at = static_cast<size_t>(head) * dk * dk;
  NarrowTile<kRuleCols> state;
  GridLaunchDependents();
  if (args.early_state) {
    LoadNarrowTile(state, seq.state + state_at, dk, tile);
  }
  GridDependencyWait();
  if (!args.early_state) {
    LoadNarrowTile(state, seq.state + state_at, dk, tile);
  }
  for (int i = lane; i < dk; i += 32) {
    sh.q[i] = seq.q[kh * dk + i];
    sh.k[i] = seq.k[kh * dk + i];
  }
  if (lane < kRuleCols) {
    sh.v[tile * kRuleCols + lane] = seq.v[head * dk + tile * kRuleCols + lane];
  }
  if (lane == 0) {
    sh.gate[0] = seq.decay[head];
    sh.gate[1] = seq.beta[head];
  }
  __syncwarp();
  float* dst = (seq.state_out != nullptr ? seq.state_out : seq.state) + state_at;
  NarrowDeltaTile(state, dst, dk, tile, sh);
  __syncwarp();
  if (lane < kRuleCols) {
    seq.y[head * dk + tile * kRuleCols + lane] = sh.y[tile * kRuleCols + lane];
  }
}

__device__ __forceinline__ float Sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float Silu(float x) { return x * Sigmoid(x); }
__device__ __forceinline__ float Softplus(float x) {
  return x > 20.0f ? x : log1pf(expf(x));
}

// Block-wide sums of two values per thread at once; results to every thread.
__device__ __forceinline__ void BlockSum2(float& a, float& b, DeltaShared& sh, int warps) {
  a = WarpSum(a);
  b = WarpSum(b);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    sh.scratch[2 * (threadIdx.x >> 5)] = a;
    sh.scratch[2 * (threadIdx.x >> 5) + 1] = b;
  }
  __syncthreads();
  a = 0.f;
  b = 0.f;
  for (int w = 0; w < warps; ++w) {
    a += sh.scratch[2 * w];
    b += sh.scratch[2 * w + 1];
  }
}

// The same for five values (the decode step's one reduction ahead of the delta
// rule: the input's sum of squares, the two gate dots, the q and k norms).
__device__ __forceinline__ void BlockSum5(float (&v)[5], DeltaShared& sh, int warps) {
#pragma unroll
  for (int i = 0; i < 5; ++i) {
    v[i] = WarpSum(v[i]);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int i = 0; i < 5; ++i) {
      sh.scratch[5 * (threadIdx.x >> 5) + i] = v[i];
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 5; ++i) {
    v[i] = 0.f;
  }
  for (int w = 0; w < warps; ++w) {
#pragma unroll
    for (int i = 0; i < 5; ++i) {
      v[i] += sh.scratch[5 * w + i];
    }
  }
}

// Mixer::Linear for one (sequence, value head). grid = (value_heads,
// sequences), 2 * dk threads: thread t < dk owns channel t of the head's q and k
// and output t of the epilogue, thread dk + t channel t of v; warp w owns columns
// 16 w .. 16 w + 15 of the state. (With dk threads and 32 columns per warp the
// kernel spent 6.5 us per layer of the decode step on four warps' worth of
// dependent instructions.)
__global__ void __launch_bounds__(2 * kDeltaThreads)
DeltaNetLinearKernel(const __grid_constant__ LinearArgs args) {
  __shared__ __align__(16) DeltaShared sh;
  const gufo_cuda_linear_seq& seq = args.seq[blockIdx.y];
  const int head = blockIdx.x;
  const int hk = args.key_heads;
  const int hv = args.value_heads;
  const int dk = args.head_dim;
  const int threads = 2 * dk;
  const int warps = threads / 32;
  const int key_dim = hk * dk;
  const int value_dim = hv * dk;
  const int channels = 2 * key_dim + value_dim;
  const int kernel = args.conv_kernel;
  const int window = kernel - 1;
  const int kh = head % hk;
  const int tid = threadIdx.x;
  const bool lower = tid < dk;        // q and k channels, the epilogue
  const int ch = lower ? tid : tid - dk;
  const float* x = seq.in;
  const size_t state_at = static_cast<size_t>(head) * dk * dk;
  NarrowTile<kStepCols> state_tile;
  // Causal depthwise conv + SiLU of a channel; also advances that channel's
  // window when this block is the one that owns it. All loads of a thread's
  // channels are issued before the first store, so they overlap.
  constexpr int kMaxWindow = 7;
  struct Taps {
    float cur;
    float old[kMaxWindow];
    float w[kMaxWindow + 1];
  };
  // The layer's weights never depend on the kernels before this one.
  auto fetch_weights = [&](int c, Taps& taps) {
    const float* kw = args.conv + static_cast<size_t>(c) * kernel;
#pragma unroll
    for (int t = 0; t < kMaxWindow; ++t) {
      if (t < window) {
        taps.w[t] = kw[t];
      }
    }
    taps.w[kMaxWindow] = kw[window];
  };
  // The window is state: written a step ago (early_state) or by the launch
  // just before this one.
  auto fetch_window = [&](int c, Taps& taps) {
#pragma unroll
    for (int t = 0; t < kMaxWindow; ++t) {
      if (t < window) {
        taps.old[t] = seq.conv_in[static_cast<size_t>(t) * channels + c];
      }
    }
  };
  auto conv = [&](int c, const Taps& taps, bool owner) -> float {
    float acc = taps.w[kMaxWindow] * taps.cur;
#pragma unroll
    for (int t = 0; t < kMaxWindow; ++t) {
      if (t < window) {
        acc = fmaf(taps.w[t], taps.old[t], acc);
        if (owner && t > 0) {
          seq.conv_out[static_cast<size_t>(t - 1) * channels + c] = taps.old[t];
        }
      }
    }
    if (owner) {
      seq.conv_out[static_cast<size_t>(window - 1) * channels + c] = taps.cur;
    }
    return Silu(acc);
  };
  // The window of the key head's q and k channels is advanced by the first
  // value head that reads the key head; every head advances its own v.
  // A lower thread convolves q (ta) and k (tb) of its channel, an upper one v (ta).
  const int ch_a = lower ? kh * dk + ch : 2 * key_dim + head * dk + ch;
  const int ch_b = key_dim + kh * dk + ch;
  Taps ta, tb;
  // The first passes of the head's alpha and beta rows (weights as well).
  constexpr int kGateAhead = 2;
  const DeltaNetGateRows& g = args.gate_rows;
  const bool gate_rows = g.alpha_w != nullptr;
  const float4* wa = reinterpret_cast<const float4*>(g.alpha_w + static_cast<size_t>(head) * g.cols);
  const float4* wb = reinterpret_cast<const float4*>(g.beta_w + static_cast<size_t>(head) * g.cols);
  float4 wa_ahead[kGateAhead], wb_ahead[kGateAhead], nw_ahead[kGateAhead];
  GridLaunchDependents();
  if (args.early_state) {
    LoadNarrowTile(state_tile, seq.ssm + state_at, dk, tid >> 5);
    fetch_window(ch_a, ta);
    if (lower) {
      fetch_window(ch_b, tb);
    }
  }
  fetch_weights(ch_a, ta);
  if (lower) {
    fetch_weights(ch_b, tb);
  }
  if (gate_rows) {
#pragma unroll
    for (int j = 0; j < kGateAhead; ++j) {
      const int i = tid + j * threads;
      if (i < g.cols / 4) {
        wa_ahead[j] = wa[i];
        wb_ahead[j] = wb[i];
        if (g.norm_w != nullptr) {
          nw_ahead[j] = reinterpret_cast<const float4*>(g.norm_w)[i];
        }
      }
    }
  }
  const float norm_w = lower ? args.ssm_norm[ch] : 0.f;
  const float ssm_a = args.ssm_a[head], dt_bias = args.dt_bias[head];
  GridDependencyWait();
  if (!args.early_state) {
    LoadNarrowTile(state_tile, seq.ssm + state_at, dk, tid >> 5);
    fetch_window(ch_a, ta);
    if (lower) {
      fetch_window(ch_b, tb);
    }
  }
  // What the epilogue needs, requested now so that it has arrived by then.
  const float z = lower ? x[channels + head * dk + ch] : 0.f;
  ta.cur = x[ch_a];
  if (lower) {
    tb.cur = x[ch_b];
  }
  if (gate_rows) {
    // The head's alpha and beta rows against the normed input, one float4 per
    // thread and pass (GgufProjections serves these F32 rows through its own
    // dot, src/models/qwen35/gguf_projections.cpp:162-170). With norm weights
    // the input is the residual stream and the RMS norm is applied on the way
    // (DeltaNetStep::Run, src/models/qwen35_2b/deltanet.cpp:358-392).
    const float* gx = args.gate_x[blockIdx.y] != nullptr ? args.gate_x[blockIdx.y] : g.x;
    const float4* xa = reinterpret_cast<const float4*>(gx);
    // The input's first passes stay in registers between the norm's sum of
    // squares and the dot products (one round trip to L2 for them, not two).
    float4 x_ahead[kGateAhead];
#pragma unroll
    for (int j = 0; j < kGateAhead; ++j) {
      const int i = tid + j * threads;
      x_ahead[j] = i < g.cols / 4 ? xa[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // One pass and one block-wide reduction: with norm weights the dots are taken
    // against x * w and scaled by the norm's 1 / rms afterwards (a scalar), so the
    // sum of squares, both dots and the q / k norms below reduce together.
    float sq = 0.f, pa = 0.f, pb = 0.f;
    auto pass = [&](float4 xv, const float4& nw, const float4& av, const float4& bv) {
      if (g.norm_w != nullptr) {
        sq += xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
        xv = make_float4(xv.x * nw.x, xv.y * nw.y, xv.z * nw.z, xv.w * nw.w);
      }
      pa += av.x * xv.x + av.y * xv.y + av.z * xv.z + av.w * xv.w;
      pb += bv.x * xv.x + bv.y * xv.y + bv.z * xv.z + bv.w * xv.w;
    };
    const float4 one4 = make_float4(1.f, 1.f, 1.f, 1.f);
#pragma unroll
    for (int j = 0; j < kGateAhead; ++j) {
      const int i = tid + j * threads;
      if (i < g.cols / 4) {
        pass(x_ahead[j], g.norm_w != nullptr ? nw_ahead[j] : one4, wa_ahead[j], wb_ahead[j]);
      }
    }
    for (int i = tid + kGateAhead * threads; i < g.cols / 4; i += threads) {
      pass(xa[i], g.norm_w != nullptr ? reinterpret_cast<const float4*>(g.norm_w)[i] : one4, wa[i], wb[i]);
    }
    float qv = 0.f, kv = 0.f;
    if (lower) {
      qv = conv(ch_a, ta, head < hk);
      kv = conv(ch_b, tb, head < hk);
    } else {
      sh.v[ch] = conv(ch_a, ta, true);
    }
    float five[5] = {sq, pa, pb, qv * qv, kv * kv};
    BlockSum5(five, sh, warps);
    const float inv = g.norm_w != nullptr ? 1.0f / sqrtf(five[0] / static_cast<float>(g.cols) + g.eps) : 1.0f;
    const float alpha = five[1] * inv, beta = five[2] * inv;
    // The two gates by two threads of the upper half.
    if (tid == dk) {
      sh.gate[0] = expf(ssm_a * Softplus(alpha + dt_bias));
    }
    if (tid == (dk >= 64 ? dk + 32 : dk)) {
      sh.gate[1] = Sigmoid(beta);
    }
    // L2 norms (+1e-6 under the root); q also takes 1/sqrt(dk).
    if (lower) {
      sh.q[ch] = qv * ((1.0f / sqrtf(five[3] + 1e-6f)) * (1.0f / sqrtf(static_cast<float>(dk))));
      sh.k[ch] = kv * (1.0f / sqrtf(five[4] + 1e-6f));
    }
  } else {
    const float* gates = x + channels + value_dim;  // alpha | beta follow z
    const float alpha = gates[head];
    const float beta = gates[hv + head];
    if (tid == dk) {
      sh.gate[0] = expf(ssm_a * Softplus(alpha + dt_bias));
    }
    if (tid == (dk >= 64 ? dk + 32 : dk)) {
      sh.gate[1] = Sigmoid(beta);
    }
    float qq = 0.f, kk = 0.f, qv = 0.f, kv = 0.f;
    if (lower) {
      qv = conv(ch_a, ta, head < hk);
      kv = conv(ch_b, tb, head < hk);
      qq = qv * qv;
      kk = kv * kv;
    } else {
      sh.v[ch] = conv(ch_a, ta, true);
    }
    BlockSum2(qq, kk, sh, warps);
    if (lower) {
      sh.q[ch] = qv * ((1.0f / sqrtf(qq + 1e-6f)) * (1.0f / sqrtf(static_cast<float>(dk))));
      sh.k[ch] = kv * (1.0f / sqrtf(kk + 1e-6f));
    }
  }
  __syncthreads();

  float* dst = (seq.ssm_out != nullptr ? seq.ssm_out : seq.ssm) + state_at;
  // (The scratch's last readers passed the barrier above.)
  NarrowDeltaTile(state_tile, dst, dk, tid >> 5, sh, &sh.scratch[tid >> 5]);
  // Gated RMSNorm over the head's dk outputs: RMS(o) * w * silu(z); the warps'
  // tiles left their outputs' squares, so one barrier serves both.
  __syncthreads();
  const float o = lower ? sh.y[ch] : 0.f;
  float total = 0.f;
  for (int w = 0; w < warps; ++w) {
    total += sh.scratch[w];
  }
  if (lower) {
    const float inv = 1.0f / sqrtf(total / static_cast<float>(dk) + args.rms_eps);
    seq.y[head * dk + ch] = o * inv * norm_w * Silu(z);
  }
}

int CheckHeads(int key_heads, int value_heads, int head_dim) {
  if (key_heads <= 0 || value_heads <= 0 || value_heads % key_heads != 0) {
    return Fail(GUFO_CUDA_SHAPE, "deltanet: value heads must tile the key heads");
  }
  if (head_dim <= 0 || head_dim > kMaxHeadDim || head_dim % 32 != 0) {
    return Fail(GUFO_CUDA_SHAPE,
                "deltanet: unsupported head dim " + std::to_string(head_dim) +
                    " (multiples of 32 up to 128)");
  }
  return GUFO_CUDA_OK;
}

}  // namespace
}  // namespace gufo

using gufo::Fail;

extern "C" {

int gufo_cuda_delta_rule_device(gufo_cuda_ctx* ctx,
                                const gufo_cuda_delta_seq* seqs, int nseq,
                                int key_heads, int value_heads, int head_dim) {
  if (ctx == nullptr || (seqs == nullptr && nseq > 0)) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "delta_rule: null pointer");
  }
  if (nseq < 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "delta_rule: negative sequence count");
  }
  int rc = gufo::CheckHeads(key_heads, value_heads, head_dim);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  for (int s = 0; s < nseq; ++s) {
    const gufo_cuda_delta_seq& q = seqs[s];
    if (q.state == nullptr || q.q == nullptr || q.k == nullptr || q.v == nullptr ||
        q.decay == nullptr || q.beta == nullptr || q.y == nullptr) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "delta_rule: null pointer in a sequence");
    }
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  for (int s0 = 0; s0 < nseq; s0 += gufo::kMaxSeqs) {
    const int n = nseq - s0 < gufo::kMaxSeqs ? nseq - s0 : gufo::kMaxSeqs;
    gufo::DeltaRuleArgs args{};
    for (int s = 0; s < n; ++s) {
      args.seq[s] = seqs[s0 + s];
    }
    args.key_heads = key_heads;
    args.value_heads = value_heads;
    args.head_dim = head_dim;
    args.early_state = ctx->early_state ? 1 : 0;
    const dim3 grid(head_dim / gufo::kRuleCols, value_heads, n);
    GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::DeltaRuleKernel, grid, dim3(32), 0,
                                         ctx->stream, 1, args));
    ctx->launches.fetch_add(1);
  }
  return GUFO_CUDA_OK;
}

int gufo_cuda_deltanet_layer_create(gufo_cuda_ctx* ctx,
                                    const gufo_cuda_deltanet_params* p,
                                    gufo_cuda_deltanet_layer* out) {
  if (ctx == nullptr || p == nullptr || out == nullptr || p->conv == nullptr ||
      p->ssm_a == nullptr || p->dt_bias == nullptr || p->ssm_norm == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_layer_create: null pointer");
  }
  int rc = gufo::CheckHeads(p->key_heads, p->value_heads, p->head_dim);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  if (p->conv_kernel < 2 || p->conv_kernel > 8) {
    return Fail(GUFO_CUDA_SHAPE, "deltanet: conv kernel must be 2..8 taps");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::DeltaNetLayer layer;
  layer.key_heads = p->key_heads;
  layer.value_heads = p->value_heads;
  layer.head_dim = p->head_dim;
  layer.conv_kernel = p->conv_kernel;
  layer.rms_eps = p->rms_eps;
  const size_t channels =
      static_cast<size_t>(2 * p->key_heads + p->value_heads) * p->head_dim;
  struct Copy {
    float** dst;
    const float* src;
    size_t n;
  } copies[] = {{&layer.conv, p->conv, channels * p->conv_kernel},
                {&layer.ssm_a, p->ssm_a, static_cast<size_t>(p->value_heads)},
                {&layer.dt_bias, p->dt_bias, static_cast<size_t>(p->value_heads)},
                {&layer.ssm_norm, p->ssm_norm, static_cast<size_t>(p->head_dim)}};
  for (auto& c : copies) {
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(c.dst), c.n * 4);
    if (e == cudaSuccess) {
      e = cudaMemcpyAsync(*c.dst, c.src, c.n * 4, cudaMemcpyHostToDevice, ctx->stream);
    }
    if (e != cudaSuccess) {
      cudaFree(layer.conv);
      cudaFree(layer.ssm_a);
      cudaFree(layer.dt_bias);
      cudaFree(layer.ssm_norm);
      return gufo::CudaFail(e, "deltanet_layer_create");
    }
  }
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  const int64_t id = ctx->next_id++;
  ctx->deltanet_layers.emplace(id, layer);
  *out = id;
  return GUFO_CUDA_OK;
}

int gufo_cuda_deltanet_layer_free(gufo_cuda_ctx* ctx,
                                  gufo_cuda_deltanet_layer layer) {
  if (ctx == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_layer_free: ctx is null");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  auto it = ctx->deltanet_layers.find(layer);
  if (it == ctx->deltanet_layers.end()) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_layer_free: unknown handle");
  }
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  cudaFree(it->second.conv);
  cudaFree(it->second.ssm_a);
  cudaFree(it->second.dt_bias);
  cudaFree(it->second.ssm_norm);
  ctx->deltanet_layers.erase(it);
  return GUFO_CUDA_OK;
}

int gufo_cuda_deltanet_linear_device(gufo_cuda_ctx* ctx,
                                     gufo_cuda_deltanet_layer layer,
                                     const gufo_cuda_linear_seq* seqs, int nseq) {
  if (ctx == nullptr || (seqs == nullptr && nseq > 0)) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_linear: null pointer");
  }
  if (nseq < 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_linear: negative sequence count");
  }
  for (int s = 0; s < nseq; ++s) {
    const gufo_cuda_linear_seq& q = seqs[s];
    if (q.in == nullptr || q.conv_in == nullptr || q.conv_out == nullptr ||
        q.ssm == nullptr || q.y == nullptr) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_linear: null pointer in a sequence");
    }
    if (q.conv_in == q.conv_out) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT,
                  "deltanet_linear: conv_in and conv_out must be distinct buffers");
    }
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  auto it = ctx->deltanet_layers.find(layer);
  if (it == ctx->deltanet_layers.end()) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_linear: unknown layer handle");
  }
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  return gufo::EnqueueDeltaNetLinear(ctx, it->second, seqs, nseq, ctx->early_state);
}

int gufo_cuda_deltanet_step_device(gufo_cuda_ctx* ctx, gufo_cuda_deltanet_layer layer, gufo_cuda_matrix ssm_alpha,
                                   gufo_cuda_matrix ssm_beta, const float* attn_norm, float rms_eps,
                                   const gufo_cuda_deltanet_step_seq* seqs, int nseq) {
  if (ctx == nullptr || attn_norm == nullptr || (seqs == nullptr && nseq > 0)) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_step: null pointer");
  }
  if (nseq < 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_step: negative sequence count");
  }
  int most = 0;
  for (int s = 0; s < nseq; ++s) {
    const gufo_cuda_deltanet_step_seq& q = seqs[s];
    if (q.n_tokens < 1 || q.n_tokens > 4) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_step: 1 to 4 tokens per sequence");
    }
    if (q.in == nullptr || q.h == nullptr || q.conv_in == nullptr || q.conv_out == nullptr || q.ssm == nullptr ||
        q.y == nullptr || (q.n_tokens >= 2 && (q.conv_saved == nullptr || q.ssm_spec == nullptr))) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_step: null pointer in a sequence");
    }
    if (q.conv_in == q.conv_out || q.conv_in == q.conv_saved || q.conv_out == q.conv_saved) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_step: the conv windows must be distinct buffers");
    }
    if ((reinterpret_cast<uintptr_t>(q.h) & 15) != 0 || q.h_stride % 4 != 0) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_step: residual rows must be 16-byte aligned");
    }
    most = q.n_tokens > most ? q.n_tokens : most;
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  auto it = ctx->deltanet_layers.find(layer);
  if (it == ctx->deltanet_layers.end()) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "deltanet_step: unknown layer handle");
  }
  const gufo::Matrix* alpha = ctx->FindMatrix(ssm_alpha);
  const gufo::Matrix* beta = ctx->FindMatrix(ssm_beta);
  if (alpha == nullptr || beta == nullptr || alpha->type != GUFO_CUDA_F32 || beta->type != GUFO_CUDA_F32 ||
      alpha->rows != it->second.value_heads || beta->rows != alpha->rows || beta->cols != alpha->cols ||
      alpha->cols % 4 != 0) {
    return Fail(GUFO_CUDA_SHAPE, "deltanet_step: ssm_alpha / ssm_beta must be F32 [hidden, value heads]");
  }
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::DeltaNetGateRows gates{};
  gates.alpha_w = reinterpret_cast<const float*>(alpha->data);
  gates.beta_w = reinterpret_cast<const float*>(beta->data);
  gates.cols = static_cast<int>(alpha->cols);
  gates.norm_w = attn_norm;
  gates.eps = rms_eps;
  // Token t of every sequence that has one, in one launch per t. Windows
  // alternate between conv_out and conv_saved so that the last token reads
  // conv_saved and writes conv_out; the last of two or more tokens leaves ssm
  // alone and writes ssm_spec.
  std::vector<gufo_cuda_linear_seq> step;
  std::vector<const float*> xs;
  for (int t = 0; t < most; ++t) {
    step.clear();
    xs.clear();
    for (int s = 0; s < nseq; ++s) {
      const gufo_cuda_deltanet_step_seq& q = seqs[s];
      if (t >= q.n_tokens) {
        continue;
      }
      const int from_end = q.n_tokens - 1 - t;   // 0 for the last token
      float* dst = from_end % 2 == 0 ? q.conv_out : q.conv_saved;
      const float* src = t == 0 ? q.conv_in : (from_end % 2 == 0 ? q.conv_saved : q.conv_out);
      const bool speculative = q.n_tokens >= 2 && from_end == 0;
      step.push_back({q.in + static_cast<size_t>(t) * q.in_stride, src, dst, q.ssm, speculative ? q.ssm_spec : nullptr,
                      q.y + static_cast<size_t>(t) * q.y_stride});
      xs.push_back(q.h + static_cast<size_t>(t) * q.h_stride);
    }
    gates.xs = xs.data();
    // States are written by the launch before this one: no early state loads.
    const int rc = gufo::EnqueueDeltaNetLinear(ctx, it->second, step.data(), static_cast<int>(step.size()), false,
                                               &gates);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
  }
  return GUFO_CUDA_OK;
}

}  // extern "C"

namespace gufo {

int EnqueueDeltaNetLinear(gufo_cuda_ctx* ctx, const DeltaNetLayer& l,
                          const gufo_cuda_linear_seq* seqs, int nseq, bool early_state,
                          const DeltaNetGateRows* gate_rows) {
  for (int s0 = 0; s0 < nseq; s0 += gufo::kMaxSeqs) {
    const int n = nseq - s0 < gufo::kMaxSeqs ? nseq - s0 : gufo::kMaxSeqs;
    gufo::LinearArgs args{};
    for (int s = 0; s < n; ++s) {
      args.seq[s] = seqs[s0 + s];
    }
    args.key_heads = l.key_heads;
    args.value_heads = l.value_heads;
    args.head_dim = l.head_dim;
    args.conv_kernel = l.conv_kernel;
    args.rms_eps = l.rms_eps;
    args.conv = l.conv;
    args.ssm_a = l.ssm_a;
    args.dt_bias = l.dt_bias;
    args.ssm_norm = l.ssm_norm;
    args.early_state = early_state ? 1 : 0;
    if (gate_rows != nullptr) {
      args.gate_rows = *gate_rows;
      for (int s = 0; s < n; ++s) {
        args.gate_x[s] = gate_rows->xs != nullptr ? gate_rows->xs[s0 + s] : nullptr;
      }
      args.gate_rows.xs = nullptr;
    }
    GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::DeltaNetLinearKernel, dim3(l.value_heads, n),
                                         dim3(2 * l.head_dim), 0, ctx->stream, 1, args));
    ctx->launches.fetch_add(1);
  }
  return GUFO_CUDA_OK;
}

}  // namespace gufo
