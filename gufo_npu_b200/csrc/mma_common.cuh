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
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

// The same with signed rows (A) as well.
__device__ __forceinline__ void MmaS8S8(int (&d)[4], const uint32_t (&a)[4],
                                        uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 "
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

// ---- bulk copies completing on a shared-memory barrier ------------------------

__device__ __forceinline__ uint32_t SharedAddress(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarArriveExpectTx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// `bytes` (a multiple of 16; both addresses 16-byte aligned) from global to this
// block's shared memory; the barrier's pending byte count drops as they land.
__device__ __forceinline__ void BulkCopy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// SM clock cycles a block waits for bytes it requested itself before giving the
// slab up (about a second; a copy that has not landed by then never will).
constexpr long long kLandLimit = 2000000000ll;

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

// Converts one 256-value block of one token into the image at `image` (shared
// or global memory): the calling warp's lane holds values 8 * lane .. + 7 of the
// block in v. Writes the three byte planes, the group sums and the column
// factors of block `b`.
__device__ __forceinline__ void StageBlock(const float (&v)[8], int lane, int tok, int b,
                                           const ImageLayout& l, uint8_t* image, float extra) {
  // Largest magnitude by integer compare of the bit patterns, so that a NaN
  // (above every finite pattern) is not lost.
  uint32_t top = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    top = max(top, __float_as_uint(v[i]) & 0x7FFFFFFFu);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    top = max(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
  }
  int e = static_cast<int>(top >> 23);  // biased exponent of the maximum
  const bool finite = e != 255;
  e = e < 22 ? 22 : e;
  // |x| < 2^(e - 126), so x * 2^(148 - e) stays below 2^22 in magnitude.
  const float up = __uint_as_float(static_cast<uint32_t>(275 - e) << 23);
  const float down = finite ? __uint_as_float(static_cast<uint32_t>(e - 21) << 23)
                            : __uint_as_float(0x7FC00000u);
  // xi + 0x808080 has the balanced digits of xi, each offset by 128, in its
  // three low bytes; flipping the offset bits leaves the signed bytes.
  uint32_t z[8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int xi = finite ? __float2int_rn(v[i] * up) : 0;
    z[i] = static_cast<uint32_t>(xi + 0x808080) ^ 0x808080u;
    sum += v[i];
  }
#pragma unroll
  for (int limb = 0; limb < kLimbs; ++limb) {
    const uint32_t pick = 0x0040u + 0x11u * limb;  // byte `limb` of both operands
    const uint32_t w0 = __byte_perm(__byte_perm(z[0], z[1], pick), __byte_perm(z[2], z[3], pick), 0x5410u);
    const uint32_t w1 = __byte_perm(__byte_perm(z[4], z[5], pick), __byte_perm(z[6], z[7], pick), 0x5410u);
    uint8_t* plane = image + static_cast<size_t>(tok * kLimbs + limb) * l.plane_stride;
    *reinterpret_cast<uint2*>(plane + b * kSuperBlock + lane * 8) = make_uint2(w0, w1);
  }
  // Group sums of the fp32 values: the lanes of one group are adjacent.
  const int lanes_per_group = l.group / 8;  // 4 (groups of 32) or 2 (of 16)
  for (int o = 1; o < lanes_per_group; o <<= 1) {
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  }
  if ((lane & (lanes_per_group - 1)) == 0) {
    float* sums = reinterpret_cast<float*>(image + l.sums_at);
    sums[static_cast<size_t>(tok) * (l.cols / l.group) + b * (kSuperBlock / l.group) +
         lane / lanes_per_group] = sum;
  }
  if (lane < kLimbs) {
    const float limb = lane == 0 ? 1.f : (lane == 1 ? 256.f : 65536.f);
    float* scale = reinterpret_cast<float*>(image + l.scale_at);
    scale[b * l.kcols + tok * kLimbs + lane] = down * limb * extra;
  }
}

__device__ __forceinline__ float SiluFast(float x) { return x * (1.0f / (1.0f + expf(-x))); }

// Builds the image of the launch's TOKENS rows in shared memory at `image` from
// the launch's fused input (prologue != kPrologueImage). Warp w converts blocks
// w, w + 8, ...; a lane holds eight adjacent values, so nothing is staged in
// between. `x` is the plain / SwiGLU input (a.x, or a group's part of it). Rows
// of several tokens follow one another: the residual, its pending add, the
// normed vector and a plain x `cols` floats apart, a SwiGLU input [gate | up]
// 2 * cols apart. A block that shares its tiles with a cluster (rank `rank` of
// `ks`, slabs of `slab_blocks` blocks dealt round-robin) converts only the
// blocks of its own slabs; the others are never read. Ends with a
// __syncthreads. kFastThreads threads.
// The norm weights of the calling warp's first block (values 8 * lane .. + 7 of
// block `warp`), for FillImage: they never depend on an earlier kernel, so a
// kernel asks for them before it waits for its predecessor (a layer's norm
// vector is read once per step: the load goes all the way to HBM, about as long
// as the whole conversion takes).
__device__ __forceinline__ void LoadNormAhead(const FastGemvArgs& a, float (&w)[8]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w[i] = 0.f;
  }
  if (a.prologue == kPrologueResNorm && warp < a.cols / kSuperBlock) {
    const float4 v0 = *reinterpret_cast<const float4*>(a.norm_w + warp * kSuperBlock + lane * 8);
    const float4 v1 = *reinterpret_cast<const float4*>(a.norm_w + warp * kSuperBlock + lane * 8 + 4);
    w[0] = v0.x, w[1] = v0.y, w[2] = v0.z, w[3] = v0.w;
    w[4] = v1.x, w[5] = v1.y, w[6] = v1.z, w[7] = v1.w;
  }
}

template <int TOKENS>
__device__ __forceinline__ void FillImage(const FastGemvArgs& a, const ImageLayout& l,
                                          uint8_t* image, float extra, const float* x,
                                          int rank, int ks, int slab_blocks, const float (&keep_w)[8]) {
  __shared__ float reduce[kFastWarps];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n = a.cols;
  const int blocks = n / kSuperBlock;
  const bool first = blockIdx.x == 0;
  auto mine = [&](int b) { return ks == 1 || (b / slab_blocks) % ks == rank; };
  auto load8 = [&](const float* p, float (&v)[8]) {
    const float4 v0 = *reinterpret_cast<const float4*>(p);
    const float4 v1 = *reinterpret_cast<const float4*>(p + 4);
    v[0] = v0.x, v[1] = v0.y, v[2] = v0.z, v[3] = v0.w;
    v[4] = v1.x, v[5] = v1.y, v[6] = v1.z, v[7] = v1.w;
  };
  auto store8 = [&](float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  };
  // Columns without a token keep a zero factor.
  float* scale = reinterpret_cast<float*>(image + l.scale_at);
  for (int i = threadIdx.x; i < blocks * l.kcols; i += kFastThreads) {
    if (i % l.kcols >= kLimbs * TOKENS) {
      scale[i] = 0.f;
    }
  }
  if (a.prologue == kPrologueResNorm) {
    // vec::RmsNorm (src/core/vec.hpp:57-63) of the residual stream after its
    // pending add (src/models/qwen35/decoder.cpp:493,504-508). The first pass
    // sums the squares; the second reads the same values again (they sit in
    // L2, and the warp's first block is still in registers).
    // keep_w: the norm weights of the warp's first block, requested by the
    // caller ahead of its dependency wait (LoadNormAhead).
#pragma unroll 1
    for (int tok = 0; tok < TOKENS; ++tok) {
      const size_t row = static_cast<size_t>(tok) * n;
      auto residual = [&](int at, float (&v)[8]) {
        load8(a.h_in + row + at, v);
        if (a.delta != nullptr) {
          // Partial sums of several ranks are added in rank order.
          const int parts = a.delta_parts > 1 ? a.delta_parts : 1;
          for (int p = 0; p < parts; ++p) {
            float d[8];
            load8(a.delta + static_cast<size_t>(p) * a.delta_stride + row + at, d);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[i] += d[i];
            }
          }
        }
      };
      if (tok > 0) {
        __syncthreads();   // the sums of the token before have been read
      }
      float keep[8] = {};
      float sq = 0.f;
      for (int b = warp; b < blocks; b += kFastWarps) {
        float v[8];
        residual(b * kSuperBlock + lane * 8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          sq = fmaf(v[i], v[i], sq);
          if (b == warp) {
            keep[i] = v[i];
          }
        }
      }
      sq = WarpSum(sq);
      if (lane == 0) {
        reduce[warp] = sq;
      }
      __syncthreads();
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kFastWarps; ++w) {
        total += reduce[w];
      }
      const float inv = 1.0f / sqrtf(total / static_cast<float>(n) + a.eps);
      for (int b = warp; b < blocks; b += kFastWarps) {
        // Block 0 writes the whole residual stream and normed vector.
        if (!first && !mine(b)) {
          continue;
        }
        const int at = b * kSuperBlock + lane * 8;
        float v[8], w[8], out[8];
        if (b == warp) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[i] = keep[i];
          }
          for (int i = 0; i < 8; ++i) {
            w[i] = keep_w[i];
          }
        } else {
          residual(at, v);
          load8(a.norm_w + at, w);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          out[i] = v[i] * inv * w[i];
        }
        if (first) {
          store8(a.h_out + row + at, v);
          if (a.normed_out != nullptr) {
            store8(a.normed_out + row + at, out);
          }
        }
        StageBlock(out, lane, tok, b, l, image, extra);
      }
    }
    if (first && threadIdx.x == 0 && a.advance != nullptr) {
      *a.advance += TOKENS;
    }
  } else {
    const size_t stride = a.prologue == kPrologueSwiGlu ? 2 * static_cast<size_t>(n) : static_cast<size_t>(n);
    const bool act = a.prologue == kPrologueSwiGlu;
    if constexpr (TOKENS == 1) {
      // A warp's blocks in batches of kBatch: all loads of a batch are in flight
      // before the first value is used (one round trip per batch, not per
      // block; a 6144-value input is three blocks per warp).
      constexpr int kBatch = 3;
      for (int b0 = warp; b0 < blocks; b0 += kBatch * kFastWarps) {
        float v[kBatch][8], up[kBatch][8];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const int b = b0 + j * kFastWarps;
          if (b < blocks && mine(b)) {
            const int at = b * kSuperBlock + lane * 8;
            load8(x + at, v[j]);
            if (act) {
              load8(x + n + at, up[j]);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const int b = b0 + j * kFastWarps;
          if (b < blocks && mine(b)) {
            if (act) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                v[j][i] = SiluFast(v[j][i]) * up[j][i];
              }
            }
            StageBlock(v[j], lane, 0, b, l, image, extra);
          }
        }
      }
    } else {
      // More tokens hold more registers elsewhere in the kernel: block by block.
#pragma unroll 1
      for (int tok = 0; tok < TOKENS; ++tok) {
        const float* xt = x + tok * stride;
        for (int b = warp; b < blocks; b += kFastWarps) {
          if (!mine(b)) {
            continue;
          }
          const int at = b * kSuperBlock + lane * 8;
          float v[8];
          load8(xt + at, v);
          if (act) {
            float up[8];
            load8(xt + n + at, up);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[i] = SiluFast(v[i]) * up[i];
            }
          }
          StageBlock(v, lane, tok, b, l, image, extra);
        }
      }
    }
  }
  __syncthreads();
}

// Tiles of 16 rows are numbered across the parts of a launch, each part
// rounded up to whole tiles.
__device__ __forceinline__ int TotalTiles(const FastGemvArgs& a) {
  int tiles = 0;
#pragma unroll
  for (int p = 0; p < kFastMaxParts; ++p) {
    if (p < a.nparts) {
      tiles += (a.parts[p].rows + 15) >> 4;
    }
  }
  return tiles;
}

// Part and tile-within-part of global tile `tile`.
__device__ __forceinline__ void LocateTile(const FastGemvArgs& a, int tile, int* part, int* local) {
  int p = 0;
#pragma unroll
  for (int i = 0; i < kFastMaxParts - 1; ++i) {
    const int tiles = (a.parts[i].rows + 15) >> 4;
    if (p == i && i + 1 < a.nparts && tile >= tiles) {
      tile -= tiles;
      p = i + 1;
    }
  }
  *part = p;
  *local = tile;
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
