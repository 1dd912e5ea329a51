// The arithmetic of one Q4_K unit (16 rows x one 256-value block) on the int8
// tensor-core path, shared by the GEMV kernel (gemv_mma.cu) and the persistent
// decode-step kernel (step_kernel.cu); the fixed-point image of the activations
// is described in mma_common.cuh. A unit is read from a slab in shared memory:
// 16 rows of up to eight 144-byte blocks, rows padded by 32 bytes so that the
// 64-bit fragment reads of the eight rows of a quarter-warp fall in distinct
// banks.
//
// MMA operand layout (m16n8k32, A row-major u8, B column-major s8). Lane
// (g = lane / 4, t = lane % 4) holds rows g and g + 8. The 32 bytes of a nibble
// pair p carry sub-block 2p in the low and 2p + 1 in the high nibbles; lane t
// loads bytes 8t..8t+7, so its two A words per row are values 8t..8t+3 and
// 8t+4..8t+7 of the sub-block and the matching B words are the same eight
// bytes of column g's plane: one 64-bit shared load, no permutation. High
// nibbles are fed as 16 q (mask 0xF0), the factor 1/16 is folded into the
// column scale.
#pragma once

#include "mma_common.cuh"

namespace gufo {
namespace q4k {

constexpr int kSlabBlocks = 8;                              // blocks per slab = warps
constexpr int kSlabRowBytes = kSlabBlocks * kQ4KBytes + 32;   // padded row in shared memory
constexpr int kSlabBytes = 16 * kSlabRowBytes;

struct Q4KUnit {
  uint4 head[2];   // rows g, g + 8: d|dmin, three scale words
  uint2 code[8];   // index 2 * pair + (0: row g, 1: row g + 8)
};

// Reads this lane's fragments of block `block` of a slab in shared memory.
__device__ __forceinline__ void LoadUnit(Q4KUnit& u, const uint8_t* slab, int block,
                                         int g, int t) {
  const uint8_t* b0 = slab + g * kSlabRowBytes + block * kQ4KBytes;
  const uint8_t* b1 = b0 + 8 * kSlabRowBytes;
  u.head[0] = *reinterpret_cast<const uint4*>(b0);
  u.head[1] = *reinterpret_cast<const uint4*>(b1);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    u.code[2 * p] = *reinterpret_cast<const uint2*>(b0 + 16 + 32 * p + 8 * t);
    u.code[2 * p + 1] = *reinterpret_cast<const uint2*>(b1 + 16 + 32 * p + 8 * t);
  }
}

// The eight 6-bit scales and mins of a block as bytes of two words each
// (quant::ScaleMinK4, src/core/quant.cpp:158-167, four sub-blocks at a time).
__device__ __forceinline__ void ScaleBytes(const uint4& h, uint32_t (&sc)[2],
                                           uint32_t (&mn)[2]) {
  sc[0] = h.y & 0x3F3F3F3Fu;
  mn[0] = h.z & 0x3F3F3F3Fu;
  sc[1] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
  mn[1] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
}

// Scale byte of sub-block J (compile time) from the two scale words.
template <int J>
__device__ __forceinline__ int ScaleOf(const uint32_t (&sc)[2]) {
  return ByteAt<(J & 3)>(sc[J >> 2]);
}

template <int TOKENS>
struct Accum {
  static constexpr int kNB = (TOKENS * kLimbs + 7) / 8;
  float out[kNB][4];     // rows g, g + 8 x columns 2t, 2t + 1
  float off[TOKENS];     // this lane's share of the dmin * m * sum(x) terms
};

// Nibble pair P of one unit: sub-blocks 2P (low nibbles) and 2P + 1 (high).
template <int TOKENS, int P>
__device__ __forceinline__ void MultiplyPair(const Q4KUnit& u, const uint32_t (&sc0)[2],
                                             const uint32_t (&sc1)[2],
                                             const uint8_t* __restrict__ at, int g,
                                             int plane_stride,
                                             int (&sum_lo)[Accum<TOKENS>::kNB][4],
                                             int (&sum_hi)[Accum<TOKENS>::kNB][4]) {
  constexpr int kNB = Accum<TOKENS>::kNB;
  constexpr int kNCols = TOKENS * kLimbs;
  const uint2 q0 = u.code[2 * P], q1 = u.code[2 * P + 1];
  const uint32_t lo[4] = {q0.x & 0x0F0F0F0Fu, q1.x & 0x0F0F0F0Fu,
                          q0.y & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu};
  const uint32_t hi[4] = {q0.x & 0xF0F0F0F0u, q1.x & 0xF0F0F0F0u,
                          q0.y & 0xF0F0F0F0u, q1.y & 0xF0F0F0F0u};
  const int s_lo0 = ScaleOf<2 * P>(sc0), s_hi0 = ScaleOf<2 * P + 1>(sc0);
  const int s_lo1 = ScaleOf<2 * P>(sc1), s_hi1 = ScaleOf<2 * P + 1>(sc1);
#pragma unroll
  for (int nb = 0; nb < kNB; ++nb) {
    // Lanes whose column holds no token read a live plane all the same: their
    // sums meet a zero column factor and are never stored.
    const uint8_t* src = at + (nb * 8 + g < kNCols ? nb * 8 * plane_stride : 0) + 64 * P;
    const uint2 xl = *reinterpret_cast<const uint2*>(src);
    const uint2 xh = *reinterpret_cast<const uint2*>(src + 32);
    int c[4];
    MmaU8S8(c, lo, xl.x, xl.y);
    sum_lo[nb][0] += s_lo0 * c[0];
    sum_lo[nb][1] += s_lo0 * c[1];
    sum_lo[nb][2] += s_lo1 * c[2];
    sum_lo[nb][3] += s_lo1 * c[3];
    MmaU8S8(c, hi, xh.x, xh.y);
    sum_hi[nb][0] += s_hi0 * c[0];
    sum_hi[nb][1] += s_hi0 * c[1];
    sum_hi[nb][2] += s_hi1 * c[2];
    sum_hi[nb][3] += s_hi1 * c[3];
  }
}

// One unit: 16 rows x one 256-value block against every staged column.
// `lane_plane` is this lane's column plane at byte 8t.
template <int TOKENS>
__device__ __forceinline__ void MultiplyUnit(const Q4KUnit& u, int b, int g, int t,
                                             const uint8_t* __restrict__ lane_plane,
                                             const ImageLayout& l,
                                             const float* __restrict__ col_scale,
                                             const float* __restrict__ sums,
                                             Accum<TOKENS>& acc) {
  constexpr int kNB = Accum<TOKENS>::kNB;
  uint32_t sc[2][2], mn[2][2];
  ScaleBytes(u.head[0], sc[0], mn[0]);
  ScaleBytes(u.head[1], sc[1], mn[1]);
  int sum_lo[kNB][4] = {}, sum_hi[kNB][4] = {};
  const uint8_t* at = lane_plane + b * kSuperBlock;
  MultiplyPair<TOKENS, 0>(u, sc[0], sc[1], at, g, l.plane_stride, sum_lo, sum_hi);
  MultiplyPair<TOKENS, 1>(u, sc[0], sc[1], at, g, l.plane_stride, sum_lo, sum_hi);
  MultiplyPair<TOKENS, 2>(u, sc[0], sc[1], at, g, l.plane_stride, sum_lo, sum_hi);
  MultiplyPair<TOKENS, 3>(u, sc[0], sc[1], at, g, l.plane_stride, sum_lo, sum_hi);
  const float d0 = HalfBitsToFloat(static_cast<uint16_t>(u.head[0].x & 0xFFFF));
  const float d1 = HalfBitsToFloat(static_cast<uint16_t>(u.head[1].x & 0xFFFF));
#pragma unroll
  for (int nb = 0; nb < kNB; ++nb) {
    const float2 cs = *reinterpret_cast<const float2*>(&col_scale[b * l.kcols + nb * 8 + 2 * t]);
    // 16 * (even sub-blocks) + (odd sub-blocks, fed as 16 q): below 2^29.
    acc.out[nb][0] = fmaf(static_cast<float>(sum_lo[nb][0] * 16 + sum_hi[nb][0]), d0 * cs.x, acc.out[nb][0]);
    acc.out[nb][1] = fmaf(static_cast<float>(sum_lo[nb][1] * 16 + sum_hi[nb][1]), d0 * cs.y, acc.out[nb][1]);
    acc.out[nb][2] = fmaf(static_cast<float>(sum_lo[nb][2] * 16 + sum_hi[nb][2]), d1 * cs.x, acc.out[nb][2]);
    acc.out[nb][3] = fmaf(static_cast<float>(sum_lo[nb][3] * 16 + sum_hi[nb][3]), d1 * cs.y, acc.out[nb][3]);
  }
  // Offsets: lanes t = 0, 1 take sub-blocks 0..3 and 4..7 of row g, lanes
  // t = 2, 3 the same of row g + 8.
  const bool second = (t >> 1) != 0;
  const bool upper = (t & 1) != 0;
  const float dmin = HalfBitsToFloat(
      static_cast<uint16_t>((second ? u.head[1].x : u.head[0].x) >> 16));
  const uint32_t m4 = second ? (upper ? mn[1][1] : mn[1][0]) : (upper ? mn[0][1] : mn[0][0]);
  const float m0 = SmallByteToFloat<0>(m4), m1 = SmallByteToFloat<1>(m4);
  const float m2 = SmallByteToFloat<2>(m4), m3 = SmallByteToFloat<3>(m4);
  const float* xs = sums + b * 8 + (upper ? 4 : 0);
#pragma unroll
  for (int k = 0; k < TOKENS; ++k) {
    const float4 s = *reinterpret_cast<const float4*>(xs + k * (l.cols / 32));
    acc.off[k] = fmaf(dmin, (m0 * s.x + m1 * s.y) + (m2 * s.z + m3 * s.w), acc.off[k]);
  }
}

}  // namespace q4k
}  // namespace gufo
