// The arithmetic of one Q6_K unit (16 rows x one 256-value block) on the int8
// tensor-core path, shared by the GEMV kernel (gemv_mma.cu) and the persistent
// decode-step kernel (step_kernel.cu); the fixed-point image of the activations
// is described in mma_common.cuh. The codes go to the MMA as the signed bytes
// 4 * (q - 32), so no offset term is left; the factor 1/4 sits in the staged
// image's column factors. A unit is read from a slab in shared memory: 16 rows
// of up to eight blocks in the planar device arrangement (common.cuh), one
// contiguous run of up to 1680 bytes per row.
//
// MMA operand layout (m16n8k32, A row-major s8, B column-major s8). A 32-value
// run (quarter k of a half) holds two scale groups: values 0..15 and 16..31.
// Lane (g, t) loads bytes 8t..8t+7 of the run's nibble and high-bit planes, so
// lanes t = 0, 1 carry the first group and t = 2, 3 the second. With several
// tokens each run is multiplied twice, against B fragments in which the other
// group's lanes read a plane of zeros; every product then holds one group's 16
// dots and takes that group's int8 scale. One token leaves room for both groups
// in the eight columns of a single product (MultiplyRun).
#pragma once

#include "mma_common.cuh"

namespace gufo {
namespace q6k {

constexpr int kSlabBlocks = kQ6KSlabBlocks;                    // blocks per slab = warps
constexpr int kSlabDataBytes = kSlabBlocks * kQ6KBytes;        // 1680
constexpr int kSlabRowBytes = kSlabDataBytes + 16;             // 424 words: 8 mod 32
constexpr int kSlabBytes = 16 * kSlabRowBytes;

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

}  // namespace q6k
}  // namespace gufo
