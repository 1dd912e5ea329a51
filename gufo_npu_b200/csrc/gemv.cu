// Dequant-fused GEMV / small-M GEMM over GGUF rows: the product behind
// Projections::Apply (GgufProjections::MatMul,
// src/models/qwen35/gguf_projections.cpp:239-286 in the reference).
//
// This file holds the general kernel: any row count, any mix of Q4_K, Q6_K and
// F32 parts in one launch, 1..8 tokens per weight read. One warp owns one
// output row; lanes split the row's blocks so that a warp reads whole 128-byte
// lines, codes are turned into fp32 once and reused for every token, and the
// sub-block scale and min are applied per 32 (Q4_K) or 16 (Q6_K) values:
//   Q4_K:  sum_j d*sc_j * (q . x)_j  -  dmin*m_j * (sum x)_j
//   Q6_K:  d * sum_g sc_g * ((q - 32) . x)_g
// fp32 accumulation throughout; lanes are combined with warp shuffles.
// HBM-bound: algorithmic bytes are the GGUF row bytes plus x and y.
#include "gemv.cuh"
#include "gemm_tc.cuh"

namespace gufo {

namespace {

template <int M>
__device__ __forceinline__ void RowQ4K(const uint8_t* __restrict__ row, int cols,
                                       const float* __restrict__ x, int lane,
                                       float (&acc)[M]) {
  const int p = lane >> 3;        // sub-block pair of this lane's word
  const int c = (lane & 7) * 4;   // first value inside the sub-blocks
  const int blocks = cols / kSuperBlock;
  for (int b = 0; b < blocks; ++b) {
    const uint32_t* block = reinterpret_cast<const uint32_t*>(row + b * kQ4KBytes);
    const uint32_t dd = __ldg(block);
    const uint32_t s0 = __ldg(block + 1), s1 = __ldg(block + 2), s2 = __ldg(block + 3);
    const uint32_t q = __ldg(block + 4 + lane);
    const float d = HalfBitsToFloat(static_cast<uint16_t>(dd & 0xFFFF));
    const float dmin = HalfBitsToFloat(static_cast<uint16_t>(dd >> 16));
    int sc_lo, m_lo, sc_hi, m_hi;
    ScaleMinK4(2 * p, s0, s1, s2, &sc_lo, &m_lo);
    ScaleMinK4(2 * p + 1, s0, s1, s2, &sc_hi, &m_hi);
    const float d_lo = d * static_cast<float>(sc_lo), o_lo = dmin * static_cast<float>(m_lo);
    const float d_hi = d * static_cast<float>(sc_hi), o_hi = dmin * static_cast<float>(m_hi);
    const float l0 = static_cast<float>(q & 0xF), l1 = static_cast<float>((q >> 8) & 0xF);
    const float l2 = static_cast<float>((q >> 16) & 0xF), l3 = static_cast<float>((q >> 24) & 0xF);
    const float h0 = static_cast<float>((q >> 4) & 0xF), h1 = static_cast<float>((q >> 12) & 0xF);
    const float h2 = static_cast<float>((q >> 20) & 0xF), h3 = static_cast<float>(q >> 28);
    const int at = b * kSuperBlock + 64 * p + c;
#pragma unroll
    for (int t = 0; t < M; ++t) {
      const float4 xl = __ldg(reinterpret_cast<const float4*>(x + static_cast<size_t>(t) * cols + at));
      const float4 xh = __ldg(reinterpret_cast<const float4*>(x + static_cast<size_t>(t) * cols + at + 32));
      const float dot_lo = l0 * xl.x + l1 * xl.y + l2 * xl.z + l3 * xl.w;
      const float dot_hi = h0 * xh.x + h1 * xh.y + h2 * xh.z + h3 * xh.w;
      const float sum_lo = (xl.x + xl.y) + (xl.z + xl.w);
      const float sum_hi = (xh.x + xh.y) + (xh.z + xh.w);
      acc[t] += d_lo * dot_lo - o_lo * sum_lo;
      acc[t] += d_hi * dot_hi - o_hi * sum_hi;
    }
  }
}

template <int M>
__device__ __forceinline__ void RowQ6K(const uint8_t* __restrict__ row, int cols,
                                       const float* __restrict__ x, int lane,
                                       float (&acc)[M]) {
  const int blocks = cols / kSuperBlock;
  for (int b = 0; b < blocks; ++b) {
    const Q6KBlock block = Q6KBlockAt(row, blocks, b);
    const float d = HalfBitsToFloat(__ldg(reinterpret_cast<const uint16_t*>(block.d)));
    float part[M];
#pragma unroll
    for (int t = 0; t < M; ++t) {
      part[t] = 0.f;
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint8_t* ql = block.ql + 64 * half;
      const uint8_t* qh = block.qh + 32 * half;
      const int8_t* sc = block.sc + 8 * half + (lane >> 4);
      const int a = __ldg(ql + lane), c = __ldg(ql + lane + 32), h = __ldg(qh + lane);
      const float w0 = static_cast<float>(static_cast<int>(__ldg(sc))) *
                       static_cast<float>(((a & 0xF) | ((h & 3) << 4)) - 32);
      const float w1 = static_cast<float>(static_cast<int>(__ldg(sc + 2))) *
                       static_cast<float>(((c & 0xF) | (((h >> 2) & 3) << 4)) - 32);
      const float w2 = static_cast<float>(static_cast<int>(__ldg(sc + 4))) *
                       static_cast<float>(((a >> 4) | (((h >> 4) & 3) << 4)) - 32);
      const float w3 = static_cast<float>(static_cast<int>(__ldg(sc + 6))) *
                       static_cast<float>(((c >> 4) | (((h >> 6) & 3) << 4)) - 32);
      const int at = b * kSuperBlock + 128 * half + lane;
#pragma unroll
      for (int t = 0; t < M; ++t) {
        const float* xt = x + static_cast<size_t>(t) * cols + at;
        part[t] += w0 * __ldg(xt) + w1 * __ldg(xt + 32) + w2 * __ldg(xt + 64) + w3 * __ldg(xt + 96);
      }
    }
#pragma unroll
    for (int t = 0; t < M; ++t) {
      acc[t] += d * part[t];
    }
  }
}

// Q5_K: Q4_K's layout with a fifth code bit per value in 32 bytes of qh
// (gguf_dot::DotK4<true>, src/models/qwen35/gguf_dot.hpp:115-193).
template <int M>
__device__ __forceinline__ void RowQ5K(const uint8_t* __restrict__ row, int cols,
                                       const float* __restrict__ x, int lane,
                                       float (&acc)[M]) {
  const int p = lane >> 3;        // sub-block pair of this lane's word
  const int c = (lane & 7) * 4;   // first value inside the sub-blocks
  const int blocks = cols / kSuperBlock;
  for (int b = 0; b < blocks; ++b) {
    const uint32_t* block = reinterpret_cast<const uint32_t*>(row + b * kQ5KBytes);
    const uint32_t dd = __ldg(block);
    const uint32_t s0 = __ldg(block + 1), s1 = __ldg(block + 2), s2 = __ldg(block + 3);
    const uint32_t h = __ldg(block + 4 + (lane & 7)) >> (2 * p);   // qh bytes c .. c + 3, this pair's bits low
    const uint32_t q = __ldg(block + 12 + lane);
    const float d = HalfBitsToFloat(static_cast<uint16_t>(dd & 0xFFFF));
    const float dmin = HalfBitsToFloat(static_cast<uint16_t>(dd >> 16));
    int sc_lo, m_lo, sc_hi, m_hi;
    ScaleMinK4(2 * p, s0, s1, s2, &sc_lo, &m_lo);
    ScaleMinK4(2 * p + 1, s0, s1, s2, &sc_hi, &m_hi);
    const float d_lo = d * static_cast<float>(sc_lo), o_lo = dmin * static_cast<float>(m_lo);
    const float d_hi = d * static_cast<float>(sc_hi), o_hi = dmin * static_cast<float>(m_hi);
    const float l0 = static_cast<float>((q & 0xF) + ((h & 1) << 4));
    const float l1 = static_cast<float>(((q >> 8) & 0xF) + (((h >> 8) & 1) << 4));
    const float l2 = static_cast<float>(((q >> 16) & 0xF) + (((h >> 16) & 1) << 4));
    const float l3 = static_cast<float>(((q >> 24) & 0xF) + (((h >> 24) & 1) << 4));
    const float h0 = static_cast<float>(((q >> 4) & 0xF) + (((h >> 1) & 1) << 4));
    const float h1 = static_cast<float>(((q >> 12) & 0xF) + (((h >> 9) & 1) << 4));
    const float h2 = static_cast<float>(((q >> 20) & 0xF) + (((h >> 17) & 1) << 4));
    const float h3 = static_cast<float>((q >> 28) + (((h >> 25) & 1) << 4));
    const int at = b * kSuperBlock + 64 * p + c;
#pragma unroll
    for (int t = 0; t < M; ++t) {
      const float4 xl = __ldg(reinterpret_cast<const float4*>(x + static_cast<size_t>(t) * cols + at));
      const float4 xh = __ldg(reinterpret_cast<const float4*>(x + static_cast<size_t>(t) * cols + at + 32));
      const float dot_lo = l0 * xl.x + l1 * xl.y + l2 * xl.z + l3 * xl.w;
      const float dot_hi = h0 * xh.x + h1 * xh.y + h2 * xh.z + h3 * xh.w;
      const float sum_lo = (xl.x + xl.y) + (xl.z + xl.w);
      const float sum_hi = (xh.x + xh.y) + (xh.z + xh.w);
      acc[t] += d_lo * dot_lo - o_lo * sum_lo;
      acc[t] += d_hi * dot_hi - o_hi * sum_hi;
    }
  }
}

// Q8_0: 32 int8 codes and one fp16 scale per 34-byte block; lane l takes value l
// of every block (gguf_dot::DotQ8_0, gguf_dot.hpp:31-69).
template <int M>
__device__ __forceinline__ void RowQ8_0(const uint8_t* __restrict__ row, int cols,
                                        const float* __restrict__ x, int lane,
                                        float (&acc)[M]) {
  const int blocks = cols / kQ8Block;
  for (int b = 0; b < blocks; ++b) {
    const uint8_t* block = row + b * kQ8Bytes;
    const float d = HalfBitsToFloat(__ldg(reinterpret_cast<const uint16_t*>(block)));
    const float w = d * static_cast<float>(static_cast<int>(static_cast<int8_t>(__ldg(block + 2 + lane))));
#pragma unroll
    for (int t = 0; t < M; ++t) {
      acc[t] = fmaf(w, __ldg(x + static_cast<size_t>(t) * cols + b * kQ8Block + lane), acc[t]);
    }
  }
}

template <int M>
__device__ __forceinline__ void RowF32(const uint8_t* __restrict__ row, int cols,
                                       const float* __restrict__ x, int lane,
                                       float (&acc)[M]) {
  const float4* w = reinterpret_cast<const float4*>(row);
  for (int i = lane; i < cols / 4; i += 32) {
    const float4 v = __ldg(w + i);
#pragma unroll
    for (int t = 0; t < M; ++t) {
      const float4 xv = __ldg(reinterpret_cast<const float4*>(x + static_cast<size_t>(t) * cols) + i);
      acc[t] += v.x * xv.x + v.y * xv.y + v.z * xv.z + v.w * xv.w;
    }
  }
}

template <int M>
__global__ void __launch_bounds__(256)
GemvRows(const __grid_constant__ GemvArgs args) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= args.total_rows) {
    return;
  }
  int p = 0;
  int local = row;
  while (p + 1 < args.nparts && local >= args.parts[p].rows) {
    local -= args.parts[p].rows;
    ++p;
  }
  const GemvPart& part = args.parts[p];
  const uint8_t* data = part.data + static_cast<size_t>(local) * part.row_bytes;
  const float* x = args.x;
  float* y = args.y;
  if (args.group_ids != nullptr) {
    const int id = args.group_ids[blockIdx.y];
    if (id < 0) {
      return;
    }
    data += static_cast<size_t>(id) * part.rows * part.row_bytes;
    x += static_cast<size_t>(blockIdx.y / (args.x_group_div > 1 ? args.x_group_div : 1)) * args.x_group_stride;
    y += static_cast<size_t>(blockIdx.y) * args.y_group_stride;
  }
  float acc[M];
#pragma unroll
  for (int t = 0; t < M; ++t) {
    acc[t] = 0.f;
  }
  if (part.type == GUFO_CUDA_Q4_K) {
    RowQ4K<M>(data, args.cols, x, lane, acc);
  } else if (part.type == GUFO_CUDA_Q6_K) {
    RowQ6K<M>(data, args.cols, x, lane, acc);
  } else if (part.type == GUFO_CUDA_Q5_K) {
    RowQ5K<M>(data, args.cols, x, lane, acc);
  } else if (part.type == GUFO_CUDA_Q8_0) {
    RowQ8_0<M>(data, args.cols, x, lane, acc);
  } else {
    RowF32<M>(data, args.cols, x, lane, acc);
  }
#pragma unroll
  for (int t = 0; t < M; ++t) {
    const float total = WarpSum(acc[t]);
    if (lane == 0) {
      y[static_cast<size_t>(t) * args.y_stride + part.out_offset + local] = total;
    }
  }
}

template <int M>
void LaunchRows(const GemvArgs& args, cudaStream_t stream) {
  const int warps = 8;
  const dim3 grid((args.total_rows + warps - 1) / warps, args.group_ids != nullptr ? args.groups : 1);
  GemvRows<M><<<grid, warps * 32, 0, stream>>>(args);
}

}  // namespace

// Enqueues y = [W_0 x | W_1 x | ...]: Q4_K and Q6_K parts on the tensor-core
// kernels (x staged once per block format, one launch per part), the rest
// together on the general kernel; at most kMaxTokens tokens per pass.
int LaunchGemv(gufo_cuda_ctx* ctx, const GemvArgs& base, int tokens) {
  if (tokens >= 16 && (reinterpret_cast<uintptr_t>(base.x) & 15) == 0) {
    // Many token rows: the parts the tcgen05 GEMM runs read their weights once
    // for all rows; the other parts take the 8-token passes below.
    GemvArgs tc = base, other = base;
    tc.nparts = other.nparts = 0;
    tc.total_rows = other.total_rows = 0;
    for (int p = 0; p < base.nparts; ++p) {
      GemvArgs& to = TcGemmRuns(ctx, base.parts[p].type, base.cols, tokens) ? tc : other;
      to.parts[to.nparts++] = base.parts[p];
      to.total_rows += base.parts[p].rows;
    }
    if (tc.nparts > 0) {
      const int rc = LaunchGemmTc(ctx, tc, tokens);
      if (rc != GUFO_CUDA_OK || other.nparts == 0) {
        return rc;
      }
      return LaunchGemv(ctx, other, tokens);
    }
  }
  for (int t0 = 0; t0 < tokens; t0 += kMaxTokens) {
    const int m = tokens - t0 < kMaxTokens ? tokens - t0 : kMaxTokens;
    const float* x = base.x + static_cast<size_t>(t0) * base.cols;
    float* y = base.y + static_cast<size_t>(t0) * base.y_stride;
    GemvArgs rest = base;
    rest.nparts = 0;
    rest.total_rows = 0;
    rest.x = x;
    rest.y = y;
    const bool fast4 = !ctx->force_general && Q4KFastFits(base.cols, m);
    const bool fast6 = !ctx->force_general && Q6KFastFits(base.cols, m);
    // Parts of one block format share one staged image and one launch.
    for (int type : {GUFO_CUDA_Q4_K, GUFO_CUDA_Q6_K}) {
      if (!(type == GUFO_CUDA_Q4_K ? fast4 : fast6)) {
        continue;
      }
      FastGemvArgs args{};
      args.cols = base.cols;
      args.y = y;
      args.y_stride = base.y_stride;
      args.tokens = m;
      // One token: every thread block stages x itself, which saves the staging
      // kernel (it reads x with 16-byte loads); more tokens share one staged image.
      const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
      args.prologue = m == 1 && aligned && !ctx->reuse_image ? kProloguePlain : kPrologueImage;
      args.x = x;
      bool staged = false;
      auto flush = [&]() -> int {
        if (args.nparts == 0) {
          return GUFO_CUDA_OK;
        }
        const int rc = type == GUFO_CUDA_Q4_K ? LaunchGemvQ4KFast(ctx, args) : LaunchGemvQ6KFast(ctx, args);
        args.nparts = 0;
        return rc;
      };
      for (int p = 0; p < base.nparts; ++p) {
        const GemvPart& part = base.parts[p];
        if (part.type != type) {
          continue;
        }
        if (args.prologue == kPrologueImage && !staged) {
          staged = true;
          // High nibbles of Q4_K reach the MMA as 16 q, Q6_K codes as 4 (q - 32): the
          // factors carry 1/16 and 1/4.
          const int rc = StageActivations(ctx, x, m, base.cols, type == GUFO_CUDA_Q4_K ? 32 : 16,
                                          type == GUFO_CUDA_Q4_K ? 1.0f / 16.0f : 0.25f, &args.image);
          if (rc != GUFO_CUDA_OK) {
            return rc;
          }
        }
        args.row_bytes = part.row_bytes;
        args.parts[args.nparts++] = {part.data, part.rows, part.out_offset};
        if (args.nparts == kFastMaxParts) {
          const int rc = flush();
          if (rc != GUFO_CUDA_OK) {
            return rc;
          }
        }
      }
      const int rc = flush();
      if (rc != GUFO_CUDA_OK) {
        return rc;
      }
    }
    for (int p = 0; p < base.nparts; ++p) {
      const GemvPart& part = base.parts[p];
      if ((fast4 && part.type == GUFO_CUDA_Q4_K) || (fast6 && part.type == GUFO_CUDA_Q6_K)) {
        continue;
      }
      rest.parts[rest.nparts++] = part;
      rest.total_rows += part.rows;
    }
    if (rest.nparts == 0) {
      continue;
    }
    switch (m) {
      case 1: LaunchRows<1>(rest, ctx->stream); break;
      case 2: LaunchRows<2>(rest, ctx->stream); break;
      case 3: LaunchRows<3>(rest, ctx->stream); break;
      case 4: LaunchRows<4>(rest, ctx->stream); break;
      case 5: LaunchRows<5>(rest, ctx->stream); break;
      case 6: LaunchRows<6>(rest, ctx->stream); break;
      case 7: LaunchRows<7>(rest, ctx->stream); break;
      default: LaunchRows<8>(rest, ctx->stream); break;
    }
    ctx->launches.fetch_add(1);
    GUFO_CUDA_TRY(cudaGetLastError());
  }
  return GUFO_CUDA_OK;
}

namespace {

// act[g][i] = silu(x[g][i]) * x[g][n + i] for the groups that run.
__global__ void __launch_bounds__(256)
SwiGluGroups(const float* __restrict__ x, int n, int x_stride, int x_div, const int* __restrict__ ids,
             float* __restrict__ act) {
  const int g = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (ids[g] < 0 || i >= n) {
    return;
  }
  const float* in = x + static_cast<size_t>(g / x_div) * x_stride;
  const float v = in[i];
  act[static_cast<size_t>(g) * n + i] = v * (1.0f / (1.0f + expf(-v))) * in[n + i];
}

}  // namespace

// Whether a grouped gate / up product can leave silu(gate) * up by itself (two
// Q4_K parts of equal whole tiles on the tensor-core kernel).
bool GroupedSwiGluInProduct(const gufo_cuda_ctx* ctx, const GemvArgs& base) {
  const bool aligned = (reinterpret_cast<uintptr_t>(base.x) & 15) == 0 && base.x_group_stride % 4 == 0;
  return !ctx->force_general && aligned && Q4KFastFits(base.cols, 1) && base.nparts == 2 &&
         base.parts[0].type == GUFO_CUDA_Q4_K && base.parts[1].type == GUFO_CUDA_Q4_K &&
         base.parts[0].rows == base.parts[1].rows && base.parts[0].rows % 16 == 0;
}

int LaunchGemvGrouped(gufo_cuda_ctx* ctx, const GemvArgs& base, int prologue, float* scratch, bool activate) {
  if (base.group_ids == nullptr || base.groups <= 0 ||
      (prologue != kProloguePlain && prologue != kPrologueSwiGlu)) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "grouped product: ids, groups and a plain or SwiGLU input");
  }
  const bool aligned = (reinterpret_cast<uintptr_t>(base.x) & 15) == 0 && base.x_group_stride % 4 == 0;
  const bool fast4 = !ctx->force_general && aligned && Q4KFastFits(base.cols, 1);
  GemvArgs rest = base;
  rest.nparts = 0;
  rest.total_rows = 0;
  FastGemvArgs args{};
  args.cols = base.cols;
  args.y = base.y;
  args.y_stride = base.y_stride;
  args.tokens = 1;
  args.prologue = prologue;
  args.x = base.x;
  args.group_ids = base.group_ids;
  args.groups = base.groups;
  args.x_group_stride = base.x_group_stride;
  args.x_group_div = base.x_group_div;
  args.y_group_stride = base.y_group_stride;
  if (activate) {
    if (!GroupedSwiGluInProduct(ctx, base)) {
      return Fail(GUFO_CUDA_UNSUPPORTED_TYPE, "grouped product: these parts cannot activate their own rows");
    }
    args.epilogue = kEpilogueSwiGlu;
  }
  for (int p = 0; p < base.nparts; ++p) {
    const GemvPart& part = base.parts[p];
    if (fast4 && part.type == GUFO_CUDA_Q4_K) {
      args.row_bytes = part.row_bytes;
      args.parts[args.nparts++] = {part.data, part.rows, part.out_offset};
      if (args.nparts == kFastMaxParts) {
        const int rc = LaunchGemvQ4KFast(ctx, args);
        if (rc != GUFO_CUDA_OK) {
          return rc;
        }
        args.nparts = 0;
      }
    } else {
      rest.parts[rest.nparts++] = part;
      rest.total_rows += part.rows;
    }
  }
  if (args.nparts > 0) {
    const int rc = LaunchGemvQ4KFast(ctx, args);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
  }
  if (rest.nparts > 0) {
    if (prologue == kPrologueSwiGlu) {
      if (scratch == nullptr) {
        return Fail(GUFO_CUDA_BAD_ARGUMENT, "grouped product: no scratch for the activated input");
      }
      SwiGluGroups<<<dim3((base.cols + 255) / 256, base.groups), 256, 0, ctx->stream>>>(
          base.x, base.cols, base.x_group_stride, base.x_group_div > 1 ? base.x_group_div : 1, base.group_ids, scratch);
      ctx->launches.fetch_add(1);
      rest.x = scratch;
      rest.x_group_stride = base.cols;
      rest.x_group_div = 1;
    }
    LaunchRows<1>(rest, ctx->stream);
    ctx->launches.fetch_add(1);
    GUFO_CUDA_TRY(cudaGetLastError());
  }
  return GUFO_CUDA_OK;
}

}  // namespace gufo

using gufo::Fail;

namespace gufo {

// Validates `parts` and fills the launch arguments; ctx->mu is held.
int BuildGemvArgs(gufo_cuda_ctx* ctx, const gufo_cuda_rows* parts, int nparts,
                  GemvArgs* args) {
  if (nparts < 1 || nparts > gufo::kMaxParts) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul: 1 to 8 parts per product");
  }
  int64_t total = 0;
  int64_t cols = 0;
  for (int p = 0; p < nparts; ++p) {
    const gufo::Matrix* m = ctx->FindMatrix(parts[p].w);
    if (m == nullptr) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul: unknown matrix handle");
    }
    if (parts[p].first < 0 || parts[p].rows <= 0 ||
        parts[p].first + parts[p].rows > m->rows) {
      return Fail(GUFO_CUDA_SHAPE, "matmul: row range outside the matrix");
    }
    if (m->type == GUFO_CUDA_F16 || m->type == GUFO_CUDA_BF16) {
      return Fail(GUFO_CUDA_UNSUPPORTED_TYPE, "matmul: F16 / BF16 rows are dequantized only, not multiplied");
    }
    if (p == 0) {
      cols = m->cols;
    } else if (m->cols != cols) {
      return Fail(GUFO_CUDA_SHAPE, "matmul: parts differ in input width");
    }
    gufo::GemvPart& out = args->parts[p];
    out.data = m->data + static_cast<size_t>(parts[p].first) * m->row_bytes;
    out.rows = static_cast<int>(parts[p].rows);
    out.out_offset = static_cast<int>(total);
    out.type = m->type;
    out.row_bytes = static_cast<int>(m->row_bytes);
    total += parts[p].rows;
  }
  if (total > INT32_MAX || cols > INT32_MAX) {
    return Fail(GUFO_CUDA_SHAPE, "matmul: product too large");
  }
  args->nparts = nparts;
  args->total_rows = static_cast<int>(total);
  args->y_stride = static_cast<int>(total);
  args->cols = static_cast<int>(cols);
  return GUFO_CUDA_OK;
}

}  // namespace gufo

extern "C" {

int gufo_cuda_matmul_device(gufo_cuda_ctx* ctx, const gufo_cuda_rows* parts,
                            int nparts, const float* device_x, int tokens,
                            float* device_y) {
  if (ctx == nullptr || parts == nullptr || device_x == nullptr || device_y == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul: null pointer");
  }
  if (tokens < 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul: negative token count");
  }
  if (reinterpret_cast<uintptr_t>(device_x) % 16 != 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul: x must be 16-byte aligned");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  gufo::GemvArgs args{};
  int rc = gufo::BuildGemvArgs(ctx, parts, nparts, &args);
  if (rc != GUFO_CUDA_OK || tokens == 0) {
    return rc;
  }
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  args.x = device_x;
  args.y = device_y;
  return gufo::LaunchGemv(ctx, args, tokens);
}

int gufo_cuda_matmul(gufo_cuda_ctx* ctx, const gufo_cuda_rows* parts, int nparts,
                     const float* host_x, int tokens, float* host_y) {
  if (ctx == nullptr || parts == nullptr || host_x == nullptr || host_y == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul: null pointer");
  }
  if (tokens < 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul: negative token count");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  gufo::GemvArgs args{};
  int rc = gufo::BuildGemvArgs(ctx, parts, nparts, &args);
  if (rc != GUFO_CUDA_OK || tokens == 0) {
    return rc;
  }
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  const size_t x_bytes = static_cast<size_t>(tokens) * args.cols * 4;
  const size_t y_bytes = static_cast<size_t>(tokens) * args.total_rows * 4;
  rc = ctx->Reserve(&ctx->stage_x, &ctx->stage_x_bytes, x_bytes);
  if (rc == GUFO_CUDA_OK) {
    rc = ctx->Reserve(&ctx->stage_y, &ctx->stage_y_bytes, y_bytes);
  }
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  GUFO_CUDA_TRY(cudaMemcpyAsync(ctx->stage_x, host_x, x_bytes, cudaMemcpyHostToDevice, ctx->stream));
  args.x = ctx->stage_x;
  args.y = ctx->stage_y;
  rc = gufo::LaunchGemv(ctx, args, tokens);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  GUFO_CUDA_TRY(cudaMemcpyAsync(host_y, ctx->stage_y, y_bytes, cudaMemcpyDeviceToHost, ctx->stream));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  return GUFO_CUDA_OK;
}

}  // extern "C"
