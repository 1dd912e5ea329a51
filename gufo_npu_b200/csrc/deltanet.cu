// The Gated DeltaNet decode step (Mixer::Linear,
// src/models/qwen35/decoder.cpp:161-265 in the reference; its delta rule,
// lines 234-257, restated blockwise in src/models/qwen35_2b/deltanet.cpp:56-82).
//
// Per value head the fp32 state S[i (key)][j (value)] is read from HBM once,
// kept on chip across the retrieval pass (u = (decay S)^T k), the rank-1 update
// (S' = decay S + k delta^T) and the readout (y = S'^T q), and written once:
// algorithmic traffic is 2 * dk * dk * 4 bytes per head, the HBM roofline of
// this kernel. Columns of S evolve independently, so a head is split into
// column tiles of kTileCols values, one thread block each; the blocks of one
// head form a thread-block cluster so that the gated RMSNorm over the head's dk
// outputs is reduced through distributed shared memory without a second pass.
//
// Thread layout (128 threads): jq = tid % 8 owns four adjacent columns (one
// float4), ig = tid / 8 owns rows ig, ig + 16, ..., so a warp's load of one
// register covers four 128-byte row segments. A thread keeps its dk/16 float4
// of S in registers between the passes; only the column sums cross threads
// (warp shuffles, then shared memory across the four warps).
#include "common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace gufo {

constexpr int kTileCols = 32;
constexpr int kDeltaThreads = 128;
constexpr int kMaxHeadDim = 128;
constexpr int kRowGroups = kDeltaThreads / 8;          // 16
constexpr int kMaxRowsPerThread = kMaxHeadDim / kRowGroups;  // 8
constexpr int kMaxSeqs = 16;                           // descriptors per launch

struct DeltaRuleArgs {
  gufo_cuda_delta_seq seq[kMaxSeqs];
  int key_heads;
  int value_heads;
  int head_dim;
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
};

namespace {

struct DeltaShared {
  float q[kMaxHeadDim];
  float k[kMaxHeadDim];
  float v[kTileCols];
  float part[kDeltaThreads / 32][kTileCols];  // per-warp column sums
  float y[kTileCols];
  float gate[2];                              // decay, beta
  float norm_part;                            // this tile's sum of y^2
  float scratch[kDeltaThreads / 32];
};

// Sums a float4 of column partials over the block's 16 row groups; every
// thread receives the total of its four columns.
__device__ __forceinline__ float4 ColumnSum(float4 v, DeltaShared& sh, int jq,
                                            int warp, int lane) {
  v.x += __shfl_xor_sync(0xFFFFFFFFu, v.x, 8);
  v.y += __shfl_xor_sync(0xFFFFFFFFu, v.y, 8);
  v.z += __shfl_xor_sync(0xFFFFFFFFu, v.z, 8);
  v.w += __shfl_xor_sync(0xFFFFFFFFu, v.w, 8);
  v.x += __shfl_xor_sync(0xFFFFFFFFu, v.x, 16);
  v.y += __shfl_xor_sync(0xFFFFFFFFu, v.y, 16);
  v.z += __shfl_xor_sync(0xFFFFFFFFu, v.z, 16);
  v.w += __shfl_xor_sync(0xFFFFFFFFu, v.w, 16);
  __syncthreads();  // the previous use of sh.part is over
  if (lane < 8) {
    *reinterpret_cast<float4*>(&sh.part[warp][4 * jq]) = v;
  }
  __syncthreads();
  float4 total = *reinterpret_cast<const float4*>(&sh.part[0][4 * jq]);
#pragma unroll
  for (int w = 1; w < kDeltaThreads / 32; ++w) {
    const float4 o = *reinterpret_cast<const float4*>(&sh.part[w][4 * jq]);
    total.x += o.x;
    total.y += o.y;
    total.z += o.z;
    total.w += o.w;
  }
  return total;
}

// The delta rule on this block's column tile. sh.q, sh.k, sh.v and sh.gate are
// ready (a __syncthreads lies between their writes and this call). Leaves the
// tile's kTileCols outputs in sh.y, visible after the trailing barrier.
struct StateTile {
  float4 s[kMaxRowsPerThread];
};

// Issues this thread's loads of the state tile; called first thing so that the
// HBM latency runs under the prologue.
__device__ __forceinline__ void LoadTile(StateTile& tile, const float* __restrict__ src,
                                         int dk, int col0) {
  const int jq = threadIdx.x & 7;
  const int ig = threadIdx.x >> 3;
  const int rows = dk / kRowGroups;
  const size_t at = static_cast<size_t>(col0 + 4 * jq);
#pragma unroll
  for (int r = 0; r < kMaxRowsPerThread; ++r) {
    if (r < rows) {
      tile.s[r] = *reinterpret_cast<const float4*>(src + static_cast<size_t>(r * kRowGroups + ig) * dk + at);
    }
  }
}

__device__ __forceinline__ void DeltaTile(StateTile& tile, float* __restrict__ dst,
                                          int dk, int col0, DeltaShared& sh) {
  const int tid = threadIdx.x;
  const int jq = tid & 7;
  const int ig = tid >> 3;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int rows = dk / kRowGroups;
  const float decay = sh.gate[0];
  const float beta = sh.gate[1];
  float4 (&s)[kMaxRowsPerThread] = tile.s;
  const size_t at = static_cast<size_t>(col0 + 4 * jq);
  // Pass 1: u_j = sum_i S_ij * (k_i * decay).
  float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < kMaxRowsPerThread; ++r) {
    if (r < rows) {
      const float ki = sh.k[r * kRowGroups + ig] * decay;
      u.x = fmaf(s[r].x, ki, u.x);
      u.y = fmaf(s[r].y, ki, u.y);
      u.z = fmaf(s[r].z, ki, u.z);
      u.w = fmaf(s[r].w, ki, u.w);
    }
  }
  u = ColumnSum(u, sh, jq, warp, lane);
  const float4 v = *reinterpret_cast<const float4*>(&sh.v[4 * jq]);
  float4 delta;
  delta.x = beta * (v.x - u.x);
  delta.y = beta * (v.y - u.y);
  delta.z = beta * (v.z - u.z);
  delta.w = beta * (v.w - u.w);
  // Pass 2: S'_ij = S_ij * decay + k_i * delta_j; y_j = sum_i S'_ij * q_i.
  float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < kMaxRowsPerThread; ++r) {
    if (r < rows) {
      const int i = r * kRowGroups + ig;
      const float ki = sh.k[i];
      const float qi = sh.q[i];
      float4 n;
      n.x = fmaf(s[r].x, decay, ki * delta.x);
      n.y = fmaf(s[r].y, decay, ki * delta.y);
      n.z = fmaf(s[r].z, decay, ki * delta.z);
      n.w = fmaf(s[r].w, decay, ki * delta.w);
      *reinterpret_cast<float4*>(dst + static_cast<size_t>(i) * dk + at) = n;
      y.x = fmaf(n.x, qi, y.x);
      y.y = fmaf(n.y, qi, y.y);
      y.z = fmaf(n.z, qi, y.z);
      y.w = fmaf(n.w, qi, y.w);
    }
  }
  y = ColumnSum(y, sh, jq, warp, lane);
  if (tid < 8) {
    *reinterpret_cast<float4*>(&sh.y[4 * jq]) = y;
  }
  __syncthreads();
}

// grid = (dk / kTileCols, value_heads, sequences); gates given.
__global__ void __launch_bounds__(kDeltaThreads)
DeltaRuleKernel(const __grid_constant__ DeltaRuleArgs args) {
  __shared__ __align__(16) DeltaShared sh;
  const gufo_cuda_delta_seq& seq = args.seq[blockIdx.z];
  const int head = blockIdx.y;
  const int dk = args.head_dim;
  const int col0 = blockIdx.x * kTileCols;
  const int kh = head % args.key_heads;
  const int tid = threadIdx.x;
  const size_t state_at = static_cast<size_t>(head) * dk * dk;
  GridLaunchDependents();
  GridDependencyWait();
  StateTile tile;
  LoadTile(tile, seq.state + state_at, dk, col0);
  if (tid < dk) {
    sh.q[tid] = seq.q[kh * dk + tid];
    sh.k[tid] = seq.k[kh * dk + tid];
  }
  if (tid < kTileCols) {
    sh.v[tid] = seq.v[head * dk + col0 + tid];
  }
  if (tid == 0) {
    sh.gate[0] = seq.decay[head];
    sh.gate[1] = seq.beta[head];
  }
  __syncthreads();
  float* dst = (seq.state_out != nullptr ? seq.state_out : seq.state) + state_at;
  DeltaTile(tile, dst, dk, col0, sh);
  if (tid < kTileCols) {
    seq.y[head * dk + col0 + tid] = sh.y[tid];
  }
}

__device__ __forceinline__ float Sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float Silu(float x) { return x * Sigmoid(x); }
__device__ __forceinline__ float Softplus(float x) {
  return x > 20.0f ? x : log1pf(expf(x));
}

// Block-wide sum of one value per thread; result to every thread.
__device__ __forceinline__ float BlockSum(float v, DeltaShared& sh) {
  v = WarpSum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    sh.scratch[threadIdx.x >> 5] = v;
  }
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kDeltaThreads / 32; ++w) {
    total += sh.scratch[w];
  }
  return total;
}

// Mixer::Linear for one (sequence, value head, column tile); the blocks of a
// head are one cluster (cluster dims = (dk / kTileCols, 1, 1)).
__global__ void __launch_bounds__(kDeltaThreads)
DeltaNetLinearKernel(const __grid_constant__ LinearArgs args) {
  __shared__ __align__(16) DeltaShared sh;
  cg::cluster_group cluster = cg::this_cluster();
  const gufo_cuda_linear_seq& seq = args.seq[blockIdx.z];
  const int head = blockIdx.y;
  const int tile = blockIdx.x;
  const int tiles = gridDim.x;
  const int hk = args.key_heads;
  const int hv = args.value_heads;
  const int dk = args.head_dim;
  const int key_dim = hk * dk;
  const int value_dim = hv * dk;
  const int channels = 2 * key_dim + value_dim;
  const int kernel = args.conv_kernel;
  const int window = kernel - 1;
  const int col0 = tile * kTileCols;
  const int kh = head % hk;
  const int tid = threadIdx.x;
  const float* x = seq.in;
  const size_t state_at = static_cast<size_t>(head) * dk * dk;
  GridLaunchDependents();
  GridDependencyWait();
  StateTile state_tile;
  LoadTile(state_tile, seq.ssm + state_at, dk, col0);

  // Causal depthwise conv + SiLU of channel ch; also advances that channel's
  // window when this block is the one that owns it.
  auto conv = [&](int ch, bool owner) -> float {
    const float* kw = args.conv + static_cast<size_t>(ch) * kernel;
    const float cur = x[ch];
    float acc = kw[window] * cur;
    for (int t = 0; t < window; ++t) {
      const float old = seq.conv_in[static_cast<size_t>(t) * channels + ch];
      acc = fmaf(kw[t], old, acc);
      if (owner && t > 0) {
        seq.conv_out[static_cast<size_t>(t - 1) * channels + ch] = old;
      }
    }
    if (owner) {
      seq.conv_out[static_cast<size_t>(window - 1) * channels + ch] = cur;
    }
    return Silu(acc);
  };
  // q and k of the key head (every tile needs all dk of each); the window of
  // those channels is advanced by the first value head that reads the key
  // head, each tile taking its own kTileCols channels.
  float qv = 0.f, kv = 0.f;
  if (tid < dk) {
    const bool owner = head < hk && tid >= col0 && tid < col0 + kTileCols;
    qv = conv(kh * dk + tid, owner);
    kv = conv(key_dim + kh * dk + tid, owner);
  }
  if (tid < kTileCols) {
    sh.v[tid] = conv(2 * key_dim + head * dk + col0 + tid, true);
  }
  // L2 norms (+1e-6 under the root); q also takes 1/sqrt(dk).
  const float qq = BlockSum(qv * qv, sh);
  const float kk = BlockSum(kv * kv, sh);
  if (tid < dk) {
    const float q_inv = 1.0f / sqrtf(qq + 1e-6f);
    const float k_inv = 1.0f / sqrtf(kk + 1e-6f);
    sh.q[tid] = qv * (q_inv * (1.0f / sqrtf(static_cast<float>(dk))));
    sh.k[tid] = kv * k_inv;
  }
  if (tid == 0) {
    const float* z_end = x + channels + value_dim;  // alpha | beta follow z
    const float alpha = z_end[head];
    const float beta = z_end[hv + head];
    sh.gate[0] = expf(args.ssm_a[head] * Softplus(alpha + args.dt_bias[head]));
    sh.gate[1] = Sigmoid(beta);
  }
  __syncthreads();

  float* dst = (seq.ssm_out != nullptr ? seq.ssm_out : seq.ssm) + state_at;
  DeltaTile(state_tile, dst, dk, col0, sh);

  // Gated RMSNorm over the head's dk outputs: RMS(o) * w * silu(z).
  float sq = 0.f;
  if (tid < kTileCols) {
    sq = sh.y[tid] * sh.y[tid];
  }
  sq = BlockSum(sq, sh);
  if (tid == 0) {
    sh.norm_part = sq;
  }
  cluster.sync();
  float total = 0.f;
  for (int r = 0; r < tiles; ++r) {
    total += *cluster.map_shared_rank(&sh.norm_part, r);
  }
  const float inv = 1.0f / sqrtf(total / static_cast<float>(dk) + args.rms_eps);
  if (tid < kTileCols) {
    const int j = col0 + tid;
    const float z = x[channels + head * dk + j];
    seq.y[head * dk + j] = sh.y[tid] * inv * args.ssm_norm[j] * Silu(z);
  }
  cluster.sync();  // peers may still be reading this block's shared memory
}

int CheckHeads(int key_heads, int value_heads, int head_dim) {
  if (key_heads <= 0 || value_heads <= 0 || value_heads % key_heads != 0) {
    return Fail(GUFO_CUDA_SHAPE, "deltanet: value heads must tile the key heads");
  }
  if (head_dim <= 0 || head_dim > kMaxHeadDim || head_dim % kTileCols != 0) {
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
    const dim3 grid(head_dim / gufo::kTileCols, value_heads, n);
    GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::DeltaRuleKernel, grid, dim3(gufo::kDeltaThreads), 0,
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
  return gufo::EnqueueDeltaNetLinear(ctx, it->second, seqs, nseq);
}

}  // extern "C"

namespace gufo {

int EnqueueDeltaNetLinear(gufo_cuda_ctx* ctx, const DeltaNetLayer& l,
                          const gufo_cuda_linear_seq* seqs, int nseq) {
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
    const int tiles = l.head_dim / gufo::kTileCols;
    GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::DeltaNetLinearKernel, dim3(tiles, l.value_heads, n),
                                         dim3(gufo::kDeltaThreads), 0, ctx->stream, tiles, args));
    ctx->launches.fetch_add(1);
  }
  return GUFO_CUDA_OK;
}

}  // namespace gufo
