// Pieces shared by the tensor-core GEMV kernels: the fixed-point image of the
// activations, its staging kernel's interface and the int8 MMA wrappers.
//
// Why integers. A decode GEMV must stay HBM-bound, which leaves about three
// issue slots per weight; turning 4- and 6-bit codes into fp32 one by one costs
// more than that. The codes are small integers, so the kernels keep them as
// bytes and let `mma.sync.m16n8k32.s32.u8.s8` (16 rows x 32 codes per issue) do
// the multiply-adds exactly, in int32. For that the fp32 activations are held
// as 24-bit fixed point per 256-value block: x = xi * 2^-shift with |xi| < 2^22,
// xi split into three signed bytes (xi = l2 * 65536 + l1 * 256 + l0), one MMA
// column per byte plane. The result is exact up to the 2^-23 (of the block's
// largest |x|) rounding of xi, the same order as fp32 accumulation; the
// per-sub-block scales are applied to the int32 sums, then one int-to-float
// conversion per 256-value block joins the fp32 accumulator of the row.
//
// The image is built once per product by StageKernel (stage.cu) in a
// context-owned device buffer and copied into shared memory by every thread
// block of the GEMV kernel that follows: a producer kernel may also write it
// directly, since it is plain memory.
#pragma once

#include "common.cuh"

namespace gufo {

constexpr int kLimbs = 3;            // byte planes per token
constexpr int kPlanePad = 32;        // bytes: plane stride = cols + 32 keeps the
                                     // 64-bit fragment reads free of bank conflicts
constexpr int kFastWarps = 8;
constexpr int kFastThreads = kFastWarps * 32;
constexpr int kMaxTokensFast = 8;    // tokens per launch (three MMA column groups)
constexpr int kFastMaxShared = 200 * 1024;

// Byte layout of the staged activations of `tokens` rows of `cols` values,
// identical in global and shared memory. Every offset is a multiple of 16.
struct ImageLayout {
  int tokens;
  int cols;
  int group;         // values per entry of `sums`: 32 (Q4_K) or 16 (Q6_K)
  int kcols;         // MMA columns, a multiple of 8 covering 3 * tokens
  int plane_stride;  // bytes between byte planes
  int scale_at;      // float [cols / 256][kcols]: 2^(8 limb - shift) * extra
  int sums_at;       // float [tokens][cols / group]: fp32 sums of x per group
  int bytes;
};

__host__ __device__ inline ImageLayout MakeImageLayout(int tokens, int cols, int group) {
  ImageLayout l;
  l.tokens = tokens;
  l.cols = cols;
  l.group = group;
  l.kcols = (tokens * kLimbs + 7) / 8 * 8;
  l.plane_stride = cols + kPlanePad;
  l.scale_at = tokens * kLimbs * l.plane_stride;
  l.sums_at = l.scale_at + (cols / kSuperBlock) * l.kcols * 4;
  l.bytes = l.sums_at + tokens * (cols / group) * 4;
  return l;
}

// Enqueues the staging of x[tokens][cols] into the context's image buffer and
// returns its device address. `extra` scales the column factors.
int StageActivations(gufo_cuda_ctx* ctx, const float* x, int tokens, int cols,
                     int group, float extra, const uint8_t** image);

__device__ __forceinline__ void MmaU8S8(int (&d)[4], const uint32_t (&a)[4],
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

// Streaming loads of weight bytes: read once, keep them out of L1.
__device__ __forceinline__ uint2 LoadStream8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
               : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 LoadStream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t LoadStream4(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Asks the memory system to bring `bytes` (a multiple of 16, 16-byte aligned
// start) into L2 without occupying registers or shared memory.
__device__ __forceinline__ void PrefetchL2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Copies `bytes` (a multiple of 16) from global to shared memory with 16-byte
// asynchronous copies spread over the block, then waits and synchronizes.
__device__ __forceinline__ void CopyImageToShared(uint8_t* dst, const uint8_t* src,
                                                  int bytes) {
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  for (int at = threadIdx.x * 16; at < bytes; at += blockDim.x * 16) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(base + at), "l"(src + at)
                 : "memory");
  }
  asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
}

// Byte `i` (compile-time) of a word, zero extended.
template <int I>
__device__ __forceinline__ int ByteAt(uint32_t w) {
  return static_cast<int>(__byte_perm(w, 0u, 0x4440u | I));
}

// Byte `I` of a word, a value below 2^23, as a float without the conversion
// pipe: the byte is placed under the exponent of 2^23 and the bias subtracted.
template <int I>
__device__ __forceinline__ float SmallByteToFloat(uint32_t w) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440u | I)) - 8388608.0f;
}

}  // namespace gufo
