// Q6_K GEMV / small-M GEMM on the int8 tensor-core path (arithmetic in
// mma_common.cuh). The product is the reference's fused Q6_K row dot
// (gguf_dot::DotQ6_K, src/models/qwen35/gguf_dot.hpp:203-290):
//   y_r = sum_blocks d * sum_g sc_g * ((q - 32) . x)_g        g = 16-value groups
// The codes go to the MMA as the signed bytes 4 * (q - 32), so no offset term
// is left; the factor 1/4 sits in the staged image's column factors.
//
// Rows are read from the planar device arrangement (common.cuh): a slab of
// eight blocks is one contiguous 1680-byte run per row, copied to shared memory
// with 16-byte asynchronous copies by the whole thread block, a ring of kStages
// slabs in flight; warp w multiplies block w of the slab. The pipeline, the persistent
// grid and the exchange of partial sums are those of the Q4_K kernel
// (gemv_q4k_mma.cu).
//
// MMA operand layout (m16n8k32, A row-major s8, B column-major s8). A 32-value
// run (quarter k of a half) holds two scale groups: values 0..15 and 16..31.
// Lane (g, t) loads bytes 8t..8t+7 of the run's nibble and high-bit planes, so
// lanes t = 0, 1 carry the first group and t = 2, 3 the second. With several
// tokens each run is multiplied twice, against B fragments in which the other
// group's lanes read a plane of zeros; every product then holds one group's 16
// dots and takes that group's int8 scale. One token leaves room for both groups
// in the eight columns of a single product (MultiplyRun).
#include <cooperative_groups.h>

#include "mma_common.cuh"

namespace gufo {
namespace {

constexpr int kSlabBlocks = kQ6KSlabBlocks;                    // blocks per slab = warps
constexpr int kSlabDataBytes = kSlabBlocks * kQ6KBytes;        // 1680
constexpr int kSlabRowBytes = kSlabDataBytes + 16;             // 424 words: 8 mod 32
constexpr int kSlabBytes = 16 * kSlabRowBytes;
constexpr int kStages = 2;

struct Q6KUnit {
  uint2 ql[2][2][2];   // [row][half][run parity]: bytes 8t..8t+7 of ql[32 * parity ..]
  uint2 qh[2][2];      // [row][half]: bytes 8t..8t+7 of qh
  uint4 sc[2];         // [row]: sixteen int8 scales
  uint32_t d[2];       // [row]: fp16 bits
};

// Reads this lane's fragments of block `j` of a slab of `n` blocks.
__device__ __forceinline__ void LoadUnit(Q6KUnit& u, const uint8_t* slab, int j, int n,
                                         int g, int t) {
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const uint8_t* row = slab + (g + 8 * r) * kSlabRowBytes;
    const uint8_t* ql = row + 128 * j + 8 * t;
    const uint8_t* qh = row + 128 * n + 64 * j + 8 * t;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      u.ql[r][half][0] = *reinterpret_cast<const uint2*>(ql + 64 * half);
      u.ql[r][half][1] = *reinterpret_cast<const uint2*>(ql + 64 * half + 32);
      u.qh[r][half] = *reinterpret_cast<const uint2*>(qh + 32 * half);
    }
    u.sc[r] = *reinterpret_cast<const uint4*>(row + 192 * n + 16 * j);
    u.d[r] = *reinterpret_cast<const uint16_t*>(row + 208 * n + 2 * j);
  }
}

template <int TOKENS>
struct Accum {
  static constexpr int kNB = (TOKENS * kLimbs + 7) / 8;
  float out[kNB][4];     // rows g, g + 8 x columns 2t, 2t + 1
  float off[TOKENS];     // this lane's share of sum_g sc_g * (sum x)_g, times d
};

// The int8 scale of group G (0..15) of a block from its four scale words.
template <int G>
__device__ __forceinline__ int ScaleOf(const uint4& sc) {
  const uint32_t w = (G >> 2) == 0 ? sc.x : ((G >> 2) == 1 ? sc.y : ((G >> 2) == 2 ? sc.z : sc.w));
  int v;
  asm("bfe.s32 %0, %1, %2, 8;" : "=r"(v) : "r"(w), "n"(8 * (G & 3)));   // sign-extending byte extract
  return v;
}

// Word W (0..3) of a block's sixteen int8 scales.
template <int W>
__device__ __forceinline__ uint32_t ScaleWord(const uint4& sc) {
  return W == 0 ? sc.x : (W == 1 ? sc.y : (W == 2 ? sc.z : sc.w));
}

// prmt with a selector whose nibbles may carry the sign-replicate bit.
__device__ __forceinline__ int SignedByte(uint32_t w, uint32_t selector) {
  int v;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(w), "r"(0u), "r"(selector));
  return v;
}

// Run K (0..3) of half H: 32 values, groups 8H + 2K and 8H + 2K + 1.
template <int TOKENS, int H, int K>
__device__ __forceinline__ void MultiplyRun(const Q6KUnit& u, const uint32_t (&hi)[2][2][4],
                                            const uint8_t* __restrict__ at_first,
                                            const uint8_t* __restrict__ at_second, int g,
                                            int stride_first, int stride_second,
                                            int (&sum)[Accum<TOKENS>::kNB][4]) {
  constexpr int kNB = Accum<TOKENS>::kNB;
  constexpr int kNCols = TOKENS * kLimbs;
  uint32_t a[4];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    // The MMA's signed byte is 4 * (code - 32): the code's low four bits at bits
    // 2..5 and its two high bits, the upper one flipped, at bits 6..7 (a 6-bit
    // two's complement number in the top of the byte).
    const uint2 q = u.ql[r][H][K & 1];
    const uint32_t lo0 = K < 2 ? (q.x << 2) : (q.x >> 2);
    const uint32_t lo1 = K < 2 ? (q.y << 2) : (q.y >> 2);
    a[r] = (lo0 & 0x3C3C3C3Cu) | hi[r][0][K];
    a[2 + r] = (lo1 & 0x3C3C3C3Cu) | hi[r][1][K];
  }
  if constexpr (TOKENS == 1) {
    // One token fills three of the eight MMA columns, so one product serves both
    // groups of the run: columns 0..2 carry the planes for values 0..15 only,
    // columns 4..6 for values 16..31 only (at_first is this lane's share of that
    // arrangement, zeros elsewhere). A lane's two output columns, 2t and 2t + 1,
    // then belong to the first group for t < 2 and to the second for t >= 2.
    const uint2 x = *reinterpret_cast<const uint2*>(at_first + 128 * H + 32 * K);
    int c[4];
    MmaS8S8(c, a, x.x, x.y);
    // The lane's group of the run is the first (t < 2) or the second; both
    // scales sit in one word, so one byte permute with the sign-replicating
    // selector (byte b to byte 0, its sign to bytes 1..3) extracts the lane's.
    const uint32_t sel = (stride_second != 0 ? 0x9991u : 0x8880u) + ((K & 1) != 0 ? 0x2222u : 0u);
    const int sg = SignedByte(ScaleWord<2 * H + (K >> 1)>(u.sc[0]), sel);
    const int sh = SignedByte(ScaleWord<2 * H + (K >> 1)>(u.sc[1]), sel);
    sum[0][0] += sg * c[0];
    sum[0][1] += sg * c[1];
    sum[0][2] += sh * c[2];
    sum[0][3] += sh * c[3];
    (void)at_second;
    (void)g;
    (void)stride_first;
  } else {
  const int s0g = ScaleOf<8 * H + 2 * K>(u.sc[0]), s1g = ScaleOf<8 * H + 2 * K + 1>(u.sc[0]);
  const int s0h = ScaleOf<8 * H + 2 * K>(u.sc[1]), s1h = ScaleOf<8 * H + 2 * K + 1>(u.sc[1]);
#pragma unroll
  for (int nb = 0; nb < kNB; ++nb) {
    // Further column groups lie 8 planes on; the plane of zeros has no such
    // neighbours (its stride is 0).
    const int hop = nb * 8 + g < kNCols ? nb * 8 : 0;
    const uint2 x0 = *reinterpret_cast<const uint2*>(at_first + hop * stride_first + 128 * H + 32 * K);
    const uint2 x1 = *reinterpret_cast<const uint2*>(at_second + hop * stride_second + 128 * H + 32 * K);
    int c[4];
    MmaS8S8(c, a, x0.x, x0.y);   // values 0..15 of the run
    sum[nb][0] += s0g * c[0];
    sum[nb][1] += s0g * c[1];
    sum[nb][2] += s0h * c[2];
    sum[nb][3] += s0h * c[3];
    MmaS8S8(c, a, x1.x, x1.y);   // values 16..31
    sum[nb][0] += s1g * c[0];
    sum[nb][1] += s1g * c[1];
    sum[nb][2] += s1h * c[2];
    sum[nb][3] += s1h * c[3];
  }
  }
}

template <int TOKENS, int H>
__device__ __forceinline__ void MultiplyHalf(const Q6KUnit& u, const uint8_t* at_first,
                                             const uint8_t* at_second, int g, int stride_first,
                                             int stride_second,
                                             int (&sum)[Accum<TOKENS>::kNB][4]) {
  // The two high bits of every code, moved to bits 6..7 with the upper one
  // flipped (code - 32 in two's complement), per row, word and run.
  uint32_t hi[2][2][4];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const uint32_t h[2] = {u.qh[r][H].x, u.qh[r][H].y};
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      hi[r][w][0] = ((h[w] << 6) & 0xC0C0C0C0u) ^ 0x80808080u;
      hi[r][w][1] = ((h[w] << 4) & 0xC0C0C0C0u) ^ 0x80808080u;
      hi[r][w][2] = ((h[w] << 2) & 0xC0C0C0C0u) ^ 0x80808080u;
      hi[r][w][3] = (h[w] & 0xC0C0C0C0u) ^ 0x80808080u;
    }
  }
  MultiplyRun<TOKENS, H, 0>(u, hi, at_first, at_second, g, stride_first, stride_second, sum);
  MultiplyRun<TOKENS, H, 1>(u, hi, at_first, at_second, g, stride_first, stride_second, sum);
  MultiplyRun<TOKENS, H, 2>(u, hi, at_first, at_second, g, stride_first, stride_second, sum);
  MultiplyRun<TOKENS, H, 3>(u, hi, at_first, at_second, g, stride_first, stride_second, sum);
}

// One unit: 16 rows x one 256-value block against every staged column.
// lane_first / lane_second: this lane's plane for the first / second group of a
// run (a plane of zeros for the group the lane does not carry).
template <int TOKENS>
__device__ __forceinline__ void MultiplyUnit(const Q6KUnit& u, int b, int g, int t,
                                             const uint8_t* __restrict__ lane_first,
                                             const uint8_t* __restrict__ lane_second,
                                             const ImageLayout& l,
                                             const float* __restrict__ col_scale,
                                             const float* __restrict__ sums,
                                             Accum<TOKENS>& acc) {
  constexpr int kNB = Accum<TOKENS>::kNB;
  int sum[kNB][4] = {};
  const uint8_t* at_first = lane_first + b * kSuperBlock;
  const uint8_t* at_second = lane_second + b * kSuperBlock;
  const int stride_first = t < 2 ? l.plane_stride : 0;
  const int stride_second = t < 2 ? 0 : l.plane_stride;
  MultiplyHalf<TOKENS, 0>(u, at_first, at_second, g, stride_first, stride_second, sum);
  MultiplyHalf<TOKENS, 1>(u, at_first, at_second, g, stride_first, stride_second, sum);
  const float d0 = HalfBitsToFloat(static_cast<uint16_t>(u.d[0]));
  const float d1 = HalfBitsToFloat(static_cast<uint16_t>(u.d[1]));
#pragma unroll
  for (int nb = 0; nb < kNB; ++nb) {
    // One token: lanes t >= 2 hold the second groups' sums of columns 2 (t - 2).
    const int col = TOKENS == 1 ? 2 * (t & 1) : nb * 8 + 2 * t;
    const float2 cs = *reinterpret_cast<const float2*>(&col_scale[b * l.kcols + col]);
    acc.out[nb][0] = fmaf(static_cast<float>(sum[nb][0]), d0 * cs.x, acc.out[nb][0]);
    acc.out[nb][1] = fmaf(static_cast<float>(sum[nb][1]), d0 * cs.y, acc.out[nb][1]);
    acc.out[nb][2] = fmaf(static_cast<float>(sum[nb][2]), d1 * cs.x, acc.out[nb][2]);
    acc.out[nb][3] = fmaf(static_cast<float>(sum[nb][3]), d1 * cs.y, acc.out[nb][3]);
  }
  // The codes went in as 4 * (code - 32): no offset term is left; the factor
  // 1/4 sits in the column scales.
  (void)sums;
}

template <int TOKENS, int PER_SM>
__global__ void __launch_bounds__(kFastThreads, PER_SM)
GemvQ6KMma(const __grid_constant__ FastGemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  // Where the blocks of a cluster leave their sums for block 0: [2][8][16][TOKENS].
  __shared__ float peers[2 * 8 * 16 * TOKENS];
  constexpr int kNB = Accum<TOKENS>::kNB;
  constexpr int kNCols = TOKENS * kLimbs;
  constexpr int kRowFloats = kNCols + TOKENS;   // per row in the exchange buffer
  constexpr int kTileFloats = 16 * kRowFloats;
  const ImageLayout l = MakeImageLayout(TOKENS, a.cols, 16);
  const int blocks = a.cols / kSuperBlock;
  const int slabs_per_tile = (blocks + kSlabBlocks - 1) / kSlabBlocks;
  const float* col_scale = reinterpret_cast<const float*>(smem + l.scale_at);
  const float* sums = reinterpret_cast<const float*>(smem + l.sums_at);
  // After the image: a plane of zeros, the exchange buffer
  // [2][warps][16 rows][kRowFloats], then the slab ring.
  uint8_t* zeros = smem + l.bytes;
  float* exchange = reinterpret_cast<float*>(zeros + l.plane_stride);
  uint8_t* ring = reinterpret_cast<uint8_t*>(exchange) + 2 * kFastWarps * kTileFloats * 4;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  // Column g of the first MMA column group; lanes past the last token's planes
  // wrap onto live ones: their sums meet a zero column factor and are never
  // stored.
  const uint8_t* plane = smem + (g % kNCols) * l.plane_stride + 8 * t;
  const uint8_t* none = zeros + 8 * t;
  // One token (see MultiplyRun): column g < 4 carries plane g for the lanes of
  // values 0..15 (t < 2), column g >= 4 carries plane g - 4 for the lanes of
  // values 16..31; columns 3 and 7 and the other lanes read zeros.
  const bool one_live = (g & 3) < kNCols && ((g < 4) == (t < 2));
  const uint8_t* lane_first = TOKENS == 1 ? (one_live ? smem + (g & 3) * l.plane_stride + 8 * t : none)
                                          : (t < 2 ? plane : none);
  const uint8_t* lane_second = t < 2 ? none : plane;
  const int row_tiles = TotalTiles(a);
  // With ksplit > 1 a cluster of ksplit blocks shares each tile.
  const int ks = a.ksplit > 1 ? a.ksplit : 1;
  const int rank = static_cast<int>(blockIdx.x) % ks;
  const int slot = static_cast<int>(blockIdx.x) / ks;
  const int stride = static_cast<int>(gridDim.x) / ks;
  const int my_tiles = (row_tiles - slot + stride - 1) / stride;
  const int slabs_mine = (slabs_per_tile - rank + ks - 1) / ks;
  const int my_slabs = my_tiles * slabs_mine;

  // Requests the next slab: warp w copies rows 2w and 2w + 1, a lane the
  // 16-byte chunks lane, lane + 32, ... of the row's run.
  const uint32_t ring_base = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
  int req_n = 0, req_s = 0;   // tile and own-slab index of the next request
  auto request = [&](int q) {
    if (q < my_slabs) {
      const int n = req_n;
      const int s = rank + req_s * ks;
      if (++req_s == slabs_mine) {
        req_s = 0;
        ++req_n;
      }
      // The row's last slab runs to the (16-byte padded) end of the row.
      const int chunks = (min(kSlabDataBytes, a.row_bytes - s * kSlabDataBytes) + 15) / 16;
      const uint32_t dst0 = ring_base + (q % kStages) * kSlabBytes;
      int part, local;
      LocateTile(a, slot + n * stride, &part, &local);
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int r = 2 * warp + rr;
        // Rows past the end repeat the last row; their sums are never stored.
        const int row = min(local * 16 + r, a.parts[part].rows - 1);
        const uint8_t* src = a.parts[part].w + static_cast<size_t>(row) * a.row_bytes + s * kSlabDataBytes;
        const uint32_t dst = dst0 + r * kSlabRowBytes;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int chunk = lane + 32 * c;
          if (chunk < chunks) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + chunk * 16),
                         "l"(src + chunk * 16) : "memory");
          }
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int q = 0; q < kStages - 1; ++q) {
    request(q);
  }
  for (int i = threadIdx.x * 16; i < l.plane_stride; i += kFastThreads * 16) {
    *reinterpret_cast<uint4*>(zeros + i) = make_uint4(0u, 0u, 0u, 0u);
  }
  GridLaunchDependents();
  // The weights above never depend on earlier kernels; the image and y do.
  GridDependencyWait();
  if (a.prologue == kPrologueImage) {
    const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    for (int at = threadIdx.x * 16; at < l.bytes; at += kFastThreads * 16) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(base + at), "l"(a.image + at)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  } else {
    FillImage<TOKENS>(a, l, smem, 0.25f, a.x, rank, ks, kSlabBlocks);
  }

  Accum<TOKENS> acc;
  auto clear = [&]() {
#pragma unroll
    for (int nb = 0; nb < kNB; ++nb) {
      acc.out[nb][0] = acc.out[nb][1] = acc.out[nb][2] = acc.out[nb][3] = 0.f;
    }
#pragma unroll
    for (int k = 0; k < TOKENS; ++k) {
      acc.off[k] = 0.f;
    }
  };
  // Sums the eight warps' partials of tile n (exchange buffer n & 1); with a
  // cluster, block 0 then adds the blocks' sums. One output per thread.
  cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
  auto gather = [&](int n) {
    int part, local;
    LocateTile(a, slot + n * stride, &part, &local);
    const int o = threadIdx.x;
    const int k = o % TOKENS;
    const int r = (o / TOKENS) & 15;
    const int row = local * 16 + r;
    const bool live = o < 16 * TOKENS && row < a.parts[part].rows;
    float total = 0.f;
    if (o < 16 * TOKENS) {
#pragma unroll
      for (int w = 0; w < kFastWarps; ++w) {
        const float* from = exchange + ((n & 1) * kFastWarps + w) * kTileFloats + r * kRowFloats;
        total += (from[k * kLimbs] + from[k * kLimbs + 1] + from[k * kLimbs + 2]) - from[kNCols + k];
      }
    }
    if (ks > 1) {
      float* slot_in_leader = cluster.map_shared_rank(peers, 0) + ((n & 1) * 8 + rank) * 16 * TOKENS;
      if (o < 16 * TOKENS) {
        slot_in_leader[o] = total;
      }
      cluster.sync();
      if (rank != 0) {
        return;
      }
      total = 0.f;
      if (o < 16 * TOKENS) {
        for (int p = 0; p < ks; ++p) {
          total += peers[((n & 1) * 8 + p) * 16 * TOKENS + o];
        }
      }
    }
    if (live) {
      a.y[static_cast<size_t>(k) * a.y_stride + a.parts[part].y_offset + row] = total;
    }
  };
  clear();
  int n = 0, s = 0;   // tile and own-slab index being multiplied
  for (int q = 0; q < my_slabs; ++q) {
    // Slab q (and, the first time, the image) has landed for this thread;
    // the barrier makes every thread's copies visible and frees slab q - 1.
    if (q == 0) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");
    }
    __syncthreads();
    request(q + kStages - 1);
    if (s == 0 && n > 0) {
      gather(n - 1);   // written before the barrier above
    }
    const int slab = rank + s * ks;
    const int b = slab * kSlabBlocks + warp;
    if (b < blocks && a.variant != 1) {
      Q6KUnit unit;
      LoadUnit(unit, ring + (q % kStages) * kSlabBytes, warp, min(kSlabBlocks, blocks - slab * kSlabBlocks), g, t);
      MultiplyUnit<TOKENS>(unit, b, g, t, lane_first, lane_second, l, col_scale, sums, acc);
    }
    if (s == slabs_mine - 1) {
      // Hand this tile's partial sums to the block.
      if constexpr (TOKENS == 1) {
        // The second groups' sums sit two lanes on, in the same columns.
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc.out[0][j] += __shfl_xor_sync(0xFFFFFFFFu, acc.out[0][j], 2);
        }
      }
      float* tile = exchange + ((n & 1) * kFastWarps + warp) * kTileFloats;
#pragma unroll
      for (int nb = 0; nb < kNB; ++nb) {
        const int col = nb * 8 + 2 * t;
        if (col < kNCols) {
          tile[g * kRowFloats + col] = acc.out[nb][0];
          tile[(g + 8) * kRowFloats + col] = acc.out[nb][2];
        }
        if (col + 1 < kNCols) {
          tile[g * kRowFloats + col + 1] = acc.out[nb][1];
          tile[(g + 8) * kRowFloats + col + 1] = acc.out[nb][3];
        }
      }
#pragma unroll
      for (int k = 0; k < TOKENS; ++k) {
        // Lanes t and t ^ 1 hold the two halves of one row's offsets.
        const float both = acc.off[k] + __shfl_xor_sync(0xFFFFFFFFu, acc.off[k], 1);
        if ((t & 1) == 0) {
          tile[(g + 8 * (t >> 1)) * kRowFloats + kNCols + k] = both;
        }
      }
      clear();
      s = 0;
      ++n;
    } else {
      ++s;
    }
  }
  if (my_tiles > 0) {
    __syncthreads();
    gather(my_tiles - 1);
  }
}

template <int TOKENS>
size_t SharedBytes(int cols) {
  const ImageLayout l = MakeImageLayout(TOKENS, cols, 16);
  return static_cast<size_t>(l.bytes) + l.plane_stride +
         static_cast<size_t>(2) * kFastWarps * 16 * (TOKENS * kLimbs + TOKENS) * 4 +
         static_cast<size_t>(kStages) * kSlabBytes;
}

template <int TOKENS>
int Launch(gufo_cuda_ctx* ctx, const FastGemvArgs& args) {
  constexpr int kPerSm = TOKENS == 1 ? 3 : 2;
  const size_t smem = SharedBytes<TOKENS>(args.cols);
  if (smem > static_cast<size_t>(kFastMaxShared)) {
    return GUFO_CUDA_TOO_LARGE;
  }
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    GUFO_CUDA_TRY(cudaFuncSetAttribute(GemvQ6KMma<TOKENS, kPerSm>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kFastMaxShared));
    configured[ctx->device & 15] = true;
  }
  int row_tiles = 0;
  for (int p = 0; p < args.nparts; ++p) {
    row_tiles += (args.parts[p].rows + 15) / 16;
  }
  if (args.group_ids != nullptr) {
    return Fail(GUFO_CUDA_UNSUPPORTED_TYPE, "fast gemv: grouped launches run Q4_K only");
  }
  // Few rows and several slabs per tile: split the tiles' slabs over a cluster.
  FastGemvArgs launch = args;
  launch.variant = ctx->gemv_variant;
  const int slabs = (args.cols / kSuperBlock + kSlabBlocks - 1) / kSlabBlocks;
  int grid = 1;
  PlanFastGrid(GemvQ6KMma<TOKENS, kPerSm>, ctx->device, kFastThreads, smem, row_tiles, slabs, &launch.ksplit, &grid);
  GUFO_CUDA_TRY(LaunchOverlapped(GemvQ6KMma<TOKENS, kPerSm>, dim3(grid), dim3(kFastThreads), smem,
                                 ctx->stream, launch.ksplit, launch));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

}  // namespace

// Whether `tokens` rows of `cols` values fit the shared-memory image.
bool Q6KFastFits(int cols, int tokens) {
  switch (tokens) {
    case 1: return SharedBytes<1>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 2: return SharedBytes<2>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 3: return SharedBytes<3>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 4: return SharedBytes<4>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 5: return SharedBytes<5>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 6: return SharedBytes<6>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 7: return SharedBytes<7>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 8: return SharedBytes<8>(cols) <= static_cast<size_t>(kFastMaxShared);
    default: return false;
  }
}

// Enqueues one Q6_K part against the staged image `args.image` (groups of 16).
int LaunchGemvQ6KFast(gufo_cuda_ctx* ctx, const FastGemvArgs& args) {
  switch (args.tokens) {
    case 1: return Launch<1>(ctx, args);
    case 2: return Launch<2>(ctx, args);
    case 3: return Launch<3>(ctx, args);
    case 4: return Launch<4>(ctx, args);
    case 5: return Launch<5>(ctx, args);
    case 6: return Launch<6>(ctx, args);
    case 7: return Launch<7>(ctx, args);
    case 8: return Launch<8>(ctx, args);
    default: return Fail(GUFO_CUDA_BAD_ARGUMENT, "fast gemv: 1 to 8 tokens per launch");
  }
}

}  // namespace gufo
