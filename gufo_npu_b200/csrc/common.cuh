// Shared declarations of the backend's translation units: the context, status
// helpers and the GGUF block decoders used by more than one kernel file.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <utility>
#include <unordered_map>
#include <vector>

#include "gufo_cuda.h"

namespace gufo {

constexpr int kSuperBlock = 256;   // values per K-quant super-block
constexpr int kQ4KBytes = 144;     // d, dmin (fp16), 12 scale bytes, 128 nibble bytes
constexpr int kQ6KBytes = 210;     // 128 ql, 64 qh, 16 int8 scales, d (fp16)
constexpr int kQ5KBytes = 176;     // d, dmin (fp16), 12 scale bytes, 32 qh, 128 nibble bytes
constexpr int kQ8Block = 32;       // values per Q8_0 block
constexpr int kQ8Bytes = 34;       // d (fp16), 32 int8

// Q6_K rows are kept on the device in a planar arrangement of the same bytes:
// GGUF blocks are 210 bytes, so inside a row they sit on 2-byte boundaries and
// neither 16-byte copies nor 4-byte fragment loads could address them. Per row
// the blocks are grouped in slabs of eight, and a slab of n blocks stores
//   ql: n x 128 | qh: n x 64 | scales: n x 16 | d: n x 2        (n x 210 bytes)
// each plane in block order. Rows start on 16-byte boundaries (the row stride
// is rounded up to a multiple of 16; padding only arises when cols / 256 is
// not a multiple of 8). quant::Dequantize's view of a block
// (src/core/quant.cpp:98-125) maps one to one: see Q6KBlock below.
constexpr int kQ6KSlabBlocks = 8;

__host__ __device__ inline size_t Q6KDeviceRowBytes(int64_t cols) {
  const size_t raw = static_cast<size_t>(cols / kSuperBlock) * kQ6KBytes;
  return (raw + 15) / 16 * 16;
}

// Device addresses of the four parts of block `b` of a planar Q6_K row.
struct Q6KBlock {
  const uint8_t* ql;
  const uint8_t* qh;
  const int8_t* sc;
  const uint8_t* d;
};

__host__ __device__ inline Q6KBlock Q6KBlockAt(const uint8_t* row, int blocks, int b) {
  const int slab = b / kQ6KSlabBlocks;
  const int j = b - slab * kQ6KSlabBlocks;
  const int left = blocks - slab * kQ6KSlabBlocks;
  const int n = left < kQ6KSlabBlocks ? left : kQ6KSlabBlocks;
  const uint8_t* base = row + static_cast<size_t>(slab) * kQ6KSlabBlocks * kQ6KBytes;
  Q6KBlock out;
  out.ql = base + 128 * j;
  out.qh = base + 128 * n + 64 * j;
  out.sc = reinterpret_cast<const int8_t*>(base + 192 * n + 16 * j);
  out.d = base + 208 * n + 2 * j;
  return out;
}

struct Matrix {
  int type = 0;
  const uint8_t* data = nullptr;  // device; Q6_K in the planar arrangement
  int64_t rows = 0;
  int64_t cols = 0;
  size_t row_bytes = 0;           // device row stride
  bool owned = false;
};

struct DeltaNetLayer {
  int key_heads = 0;
  int value_heads = 0;
  int head_dim = 0;
  int conv_kernel = 0;
  float rms_eps = 0;
  float* conv = nullptr;      // device copies
  float* ssm_a = nullptr;
  float* dt_bias = nullptr;
  float* ssm_norm = nullptr;
};

struct DeltaNetLayer;
void SetError(const std::string& text);
int Fail(int status, const std::string& text);
int CudaFail(cudaError_t e, const char* what);

// How a tensor-core GEMV obtains its input vector. The fused forms mirror the
// prologues of the reference's NPU GEMV (npu::Prologue kPlain / kAct /
// kResNorm, src/npu/gemv.hpp:58-63): they remove a kernel boundary, not a
// weight read.
enum FastPrologue {
  kPrologueImage = 0,    // a fixed-point image staged earlier (any token count)
  kProloguePlain = 1,    // x fp32 rows, staged by every thread block
  kPrologueResNorm = 2,  // x = RMS(h_in + delta) * norm_w; block 0 also writes h_out and normed_out
  kPrologueSwiGlu = 3,   // x[i] = silu(x_in[i]) * x_in[cols + i]
};

constexpr int kFastMaxParts = 4;
constexpr int kEpilogueSwiGlu = 1;
constexpr int kMaxPeers = 8;

// Row-split ranks (peer.cu). A product with `world` > 0 stores its rows into
// every rank's copy of the full vector and, when its last thread block is
// done, raises this rank's flag of the vector's slot in every rank's arena.
struct PeerOut {
  int world;
  int rank;
  int slot;
  float* y[kMaxPeers];          // where this rank's rows start in rank p's arena
  unsigned* header[kMaxPeers];  // the arenas' headers (flags, counters)
};
// A kernel whose input is such a vector waits (bounded) until every rank's
// flag of the slot has reached the turn this rank's own product announced.
struct PeerWait {
  const unsigned* header;       // this rank's arena header; null: no wait
  int world;
  int slot;
  long long limit;              // clock cycles
};

struct FastPart {
  const uint8_t* w;   // first row
  int rows;
  int y_offset;       // column of y where this part starts
};

// One launch of a tensor-core GEMV kernel: parts of one block format sharing
// one input.
struct FastGemvArgs {
  FastPart parts[kFastMaxParts];
  int nparts;
  int cols;
  int row_bytes;
  float* y;              // [tokens][y_stride]
  int y_stride;
  int tokens;            // rows of x and y (grouped launches: 1)
  int prologue;
  const uint8_t* image;  // kPrologueImage
  const float* x;        // kProloguePlain: [tokens][cols]; kPrologueSwiGlu: [tokens][2 * cols]
  const float* h_in;     // kPrologueResNorm: the residual stream [tokens][cols] ...
  const float* delta;    //   ... plus this, [tokens][cols] (may be null)
  int delta_parts;       //   ... and delta_parts - 1 more such vectors, delta_stride floats apart,
  int delta_stride;      //   added in order (0 or 1: the one vector; one token only otherwise)
  const float* norm_w;
  float eps;
  float* h_out;          //   h_in + delta, written by block 0 (must not alias h_in)
  float* normed_out;     //   the normed rows, written by block 0 (may be null)
  int* advance;          //   incremented by `tokens` by block 0 (may be null)
  // Thread blocks per 16-row tile (a cluster): block r of a cluster takes the
  // slabs r, r + ksplit, ... and the partial sums meet in block 0's shared
  // memory. Set by the launcher for matrices with few rows.
  int ksplit;
  int tiles_each;         // set by the launcher: with ksplit == 1 block b multiplies tiles_each tiles,
  int tiles_more;         //   one more if b < tiles_more
  // Grouped launches (the routed experts of a MoE layer): the parts are stacks
  // of `rows`-row matrices, group g multiplies matrix group_ids[g] of every
  // part (a negative id skips the group) with its own input and output. The
  // ids live on the device, so a router kernel can feed the launch directly.
  const int* group_ids;   // null: one ungrouped product
  int groups;
  int x_group_stride;     // floats between the inputs (0: shared)
  int x_group_div;        // groups per input: group g reads input g / x_group_div (0 counts as 1)
  // Timing experiments (context option "gemv_variant"; wrong results): 1 skips
  // the multiplies and leaves only the data movement.
  int variant;
  int y_group_stride;     // floats between the groups' outputs
  // kEpilogueSwiGlu: the two parts are the gate and up rows of an FFN (equal row
  // counts, whole tiles); every block multiplies tile t of both and stores
  // act[t] = silu(gate[t]) * up[t] as rows/part outputs per token, y_stride
  // apart (npu::Epilogue::kSwiGlu, src/npu/gemv.hpp:64-68). The launcher gives
  // every tile pair a block of its own.
  int epilogue;
  PeerOut peer_out;       // world == 0: an ordinary product
  PeerWait peer_wait;
};

// A single-part launch against a staged image.
inline FastGemvArgs ImageGemvArgs(const uint8_t* w, int rows, int cols, int row_bytes,
                                  const uint8_t* image, float* y, int y_stride, int y_offset,
                                  int tokens) {
  FastGemvArgs a{};
  a.parts[0] = {w, rows, y_offset};
  a.nparts = 1;
  a.cols = cols;
  a.row_bytes = row_bytes;
  a.y = y;
  a.y_stride = y_stride;
  a.tokens = tokens;
  a.prologue = kPrologueImage;
  a.image = image;
  return a;
}

// Bytes of a row of `cols` values of `type`; 0 when the type is not run here or
// cols is not a whole number of blocks.
size_t RowBytes(int type, int64_t cols);
// Device row stride of a matrix of `type` (differs from RowBytes for Q6_K rows
// whose GGUF size is not a multiple of 16).
size_t DeviceRowBytes(int type, int64_t cols);

}  // namespace gufo

struct gufo_cuda_ctx;
namespace gufo {
// Enqueues one Q4_K part on the int8 tensor-core kernel against a staged image.
int LaunchGemvQ4KFast(gufo_cuda_ctx* ctx, const FastGemvArgs& args);
// Whether the image of `tokens` rows of `cols` values fits in shared memory.
bool Q4KFastFits(int cols, int tokens);
bool FastSwiGluPairsFit(const gufo_cuda_ctx* ctx, int type, int cols, int tokens, int pairs);
// One Mixer::Linear step per sequence; the caller holds ctx->mu.
// `early_state`: the states and conv windows were not written by the kernels
// shortly before this one in the stream (several may be in flight at once), so
// their loads may run ahead of the dependency wait.
// The F32 alpha / beta rows of a DeltaNet layer's input product, for a step
// that computes the two gates inside the mixer kernel instead of reading them
// from the product's output: a = alpha_w[head] . x, b = beta_w[head] . x.
struct DeltaNetGateRows {
  const float* x;         // the layer's normed input [cols] (every sequence's, unless xs is given)
  const float* alpha_w;   // [value heads][cols]
  const float* beta_w;
  int cols;               // a multiple of 4
  // Non-null norm_w: x holds the residual stream instead and the kernel applies
  // vec::RmsNorm (src/core/vec.hpp:57-63) with these weights first.
  const float* norm_w;
  float eps;
  // Per-sequence inputs (launch order), overriding x when non-null.
  const float* const* xs;
};
int EnqueueDeltaNetLinear(gufo_cuda_ctx* ctx, const DeltaNetLayer& layer,
                          const gufo_cuda_linear_seq* seqs, int nseq, bool early_state,
                          const DeltaNetGateRows* gate_rows = nullptr);
// The same for Q6_K parts (image with group sums of 16).
int LaunchGemvQ6KFast(gufo_cuda_ctx* ctx, const FastGemvArgs& args);
bool Q6KFastFits(int cols, int tokens);
}  // namespace gufo

struct gufo_cuda_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int sm_count = 0;
  std::mutex mu;
  std::unordered_map<int64_t, gufo::Matrix> matrices;
  std::unordered_map<int64_t, gufo::DeltaNetLayer> deltanet_layers;
  int64_t next_id = 1;
  // Staging for the host-pointer entry points.
  float* stage_x = nullptr;
  size_t stage_x_bytes = 0;
  float* stage_y = nullptr;
  size_t stage_y_bytes = 0;
  // Fixed-point image of the activations of the product in flight.
  uint8_t* image = nullptr;
  size_t image_bytes = 0;
  // Scratch of the tcgen05 GEMM: an error word, the fp16 activation tile
  // images, the partial sums of split products.
  uint8_t* tc_scratch = nullptr;
  size_t tc_scratch_bytes = 0;
  // Scratch blocks that were outgrown: a CUDA graph captured earlier may still
  // hold their addresses, so they stay allocated until the context goes.
  std::vector<void*> retired;
  // Products of 16 or more token rows run on the tcgen05 GEMM (option "tc_gemm").
  bool tc_gemm = true;
  bool tc_gemm_all = false;   // option value 2: from 16 rows on, whatever is faster
  std::atomic<int64_t> launches{0};
  // Test hook: route every product through the general kernel.
  bool force_general = false;
  // Timing hook: skip the staging kernel and multiply against the image of the
  // previous product (wrong results unless x is unchanged).
  bool reuse_image = false;
  int gemv_variant = 0;
  // The caller's promise that DeltaNet states passed to this context were not
  // written by the two kernels enqueued just before the call.
  bool early_state = false;
  // One-token steps of a resident decoder run as one persistent kernel where
  // the model allows it and this is set (option "step_kernel"). Off unless
  // asked for: on B200 a grid-wide barrier costs as much as a programmatic
  // kernel boundary, and the launch chain is the faster of the two.
  bool step_kernel = false;
  // How long a wait inside that kernel may take (option "step_wait_us").
  int64_t step_wait_us = 2000000;
  // Test hook (option "step_skip_arrival"): block 0 stays away from the grid
  // barrier after this operation, so that the others' waits run out (-1: off).
  int step_skip_arrival = -1;

  const gufo::Matrix* FindMatrix(int64_t id) const {
    auto it = matrices.find(id);
    return it == matrices.end() ? nullptr : &it->second;
  }
  int Reserve(float** buffer, size_t* have, size_t want);
  // Grows a device scratch block to `want` bytes (at least `floor`) without
  // freeing the old one and without waiting for the stream; refuses while the
  // stream is being captured (a capture cannot allocate). ctx->mu is held.
  int GrowScratch(uint8_t** block, size_t* have, size_t want, size_t floor, const char* what);
};

#define GUFO_CUDA_TRY(expr)                                 \
  do {                                                      \
    cudaError_t gufo_e_ = (expr);                           \
    if (gufo_e_ != cudaSuccess) {                           \
      return gufo::CudaFail(gufo_e_, #expr);                \
    }                                                       \
  } while (0)

namespace gufo {

// Launches `kernel` so that it may begin while the previous kernel in the
// stream is still draining (programmatic dependent launch). Such a kernel must
// execute GridDependencyWait() before it reads anything an earlier kernel
// wrote and before its first global write. `cluster_x` > 1 also groups the
// grid's x dimension into thread-block clusters.
template <typename... KernelArgs, typename... Args>
cudaError_t LaunchOverlapped(void (*kernel)(KernelArgs...), dim3 grid, dim3 block,
                             size_t smem, cudaStream_t stream, int cluster_x,
                             Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[n].val.programmaticStreamSerializationAllowed = 1;
  ++n;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  config.attrs = attr;
  config.numAttrs = n;
  return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

// How many blocks of `kernel` (in clusters of `cluster_x`) the device holds at
// once with `smem` bytes of dynamic shared memory each. Asked of the runtime
// once per (device, smem, cluster) and remembered; 0 when the query fails.
template <typename Kernel>
int ResidentBlocks(Kernel kernel, int device, int threads, size_t smem, int cluster_x) {
  struct Entry {
    int device;
    size_t smem;
    int cluster;
    int blocks;
  };
  static Entry cache[32];
  static int cached = 0;
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  for (int i = 0; i < cached; ++i) {
    if (cache[i].device == device && cache[i].smem == smem && cache[i].cluster == cluster_x) {
      return cache[i].blocks;
    }
  }
  int blocks = 0;
  if (cluster_x > 1) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(cluster_x * 64);
    config.blockDim = dim3(threads);
    config.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = cluster_x;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    config.attrs = &attr;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
      cudaGetLastError();
      clusters = 0;
    }
    blocks = clusters * cluster_x;
  } else {
    int per_sm = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
      cudaGetLastError();
      per_sm = 0;
    }
    blocks = per_sm * sms;
  }
  if (cached < 32) {
    cache[cached++] = Entry{device, smem, cluster_x, blocks};
  }
  return blocks;
}

// Picks how many blocks share a tile's slabs (1, 2, 3 or 4: the largest that
// still lets every tile run at once) and the grid for it.
template <typename Kernel>
void PlanFastGrid(Kernel kernel, int device, int threads, size_t smem, int row_tiles, int slabs,
                  int* ksplit, int* grid) {
  for (int ks = slabs < 4 ? slabs : 4; ks >= 2; --ks) {
    const int resident = ResidentBlocks(kernel, device, threads, smem, ks);
    if (row_tiles * ks <= resident) {
      *ksplit = ks;
      *grid = row_tiles * ks;
      return;
    }
  }
  int resident = ResidentBlocks(kernel, device, threads, smem, 1);
  if (resident <= 0) {
    resident = 1;
  }
  *ksplit = 1;
  *grid = row_tiles < resident ? row_tiles : resident;
}

// ---- device helpers ------------------------------------------------------

// Lets the next kernel of the stream start launching its blocks.
__device__ __forceinline__ void GridLaunchDependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// Waits until every earlier kernel of the stream has finished and its writes
// are visible.
__device__ __forceinline__ void GridDependencyWait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// fp16 bits to fp32, exact for every input including subnormals (the
// conversion quant::HalfToFloat spells out, src/core/quant.cpp:129-155).
__device__ __forceinline__ float HalfBitsToFloat(uint16_t h) {
  float f;
  asm("{ .reg .b16 t; mov.b16 t, %1; cvt.f32.f16 %0, t; }" : "=f"(f) : "h"(h));
  return f;
}

// The 6-bit scale and min of sub-block j of a Q4_K block from its 12 packed
// bytes held as three little-endian words (quant::ScaleMinK4,
// src/core/quant.cpp:158-167).
__device__ __forceinline__ void ScaleMinK4(int j, uint32_t s0, uint32_t s1,
                                           uint32_t s2, int* sc, int* m) {
  const int shift = 8 * (j & 3);
  const uint32_t a = (s0 >> shift) & 0xFFu;  // bytes 0..3
  const uint32_t b = (s1 >> shift) & 0xFFu;  // bytes 4..7
  if (j < 4) {
    *sc = a & 63;
    *m = b & 63;
  } else {
    const uint32_t c = (s2 >> shift) & 0xFFu;  // bytes 8..11
    *sc = (c & 0x0F) | ((a >> 6) << 4);
    *m = (c >> 4) | ((b >> 6) << 4);
  }
}

__device__ __forceinline__ float WarpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  }
  return v;
}

}  // namespace gufo
