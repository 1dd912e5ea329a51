// Dequant-fused small-M GEMM on the fifth-generation tensor cores: the product
// behind Projections::Apply (GgufProjections::MatMul,
// src/models/qwen35/gguf_projections.cpp:239-286 in the reference) when 16 to
// 128 token rows share one weight read - the ragged verify batch, where every
// sequence brings a few draft tokens and the packed rows form one matrix.
//
// One thread block multiplies 128 weight rows by all the tokens:
//   D[128 rows][N tokens] (fp32, tensor memory) += A[128][64] * B[N][64]^T
// per 64 columns, with A the weights as fp16 and B the activations as fp16.
//   - loader warp: bulk copies (cp.async.bulk, completion on an mbarrier) bring
//     the rows' Q4_K blocks (144 B each) and the activation tiles into shared
//     memory; the activations were converted once per product into tile images
//     that already carry the shared-memory swizzle, so a tile is one copy;
//   - four dequant warps, one thread per weight row: w = d*sc*q - dmin*m in fp32
//     (DequantQ4_K, src/core/quant.cpp:33-59), rounded once to fp16 and stored
//     in the 128-byte-swizzled K-major layout the MMA reads;
//   - one thread issues tcgen05.mma (kind::f16, M = 128, N = tokens rounded to
//     16, K = 16, four per tile) and tcgen05.commit hands the tile buffers back;
//   - the dequant warps then read the accumulator with tcgen05.ld and store
//     y[token][row], 32 consecutive rows per warp store.
// Each activation row is scaled by a power of two into fp16 range first and the
// outputs scaled back, so range never costs precision. Rounding w and x to
// fp16 (11 significant bits) bounds the relative L2 error of y near 2e-4.
//
// Roofline: weights stream once from HBM (0.5625 B per weight); 2 * 128 * N * 64
// flops per tile. Below N ~ 64 the bound is HBM (and the dequant arithmetic,
// about 4 instructions per weight); above it the tensor pipe.
// Matrices with few rows split K over several thread blocks; their partial
// sums are added in a fixed order by a second kernel.
//
// Every wait on an mbarrier is bounded: a wait that runs out records an error
// code, raises a block-wide abort flag that ends all other waits, and the
// kernel still frees its tensor memory and returns.
#include "gemm_tc.cuh"

#include <cuda_fp16.h>

namespace gufo {

namespace {

constexpr int kTileRows = 128;
constexpr int kTileK = 64;                 // values per A / B tile (one swizzle row of fp16)
constexpr int kTileBytes = kTileRows * kTileK * 2;   // 16 KiB
constexpr int kAbStages = 4;
constexpr int kRawStages = 3;
constexpr int kRawBytes = kTileRows * kQ4KBytes;     // one Q4_K block of every row
constexpr int kDequantThreads = 128;
constexpr int kTcThreads = kDequantThreads + 64;     // + loader warp + MMA warp
constexpr int kTmemColumns = 128;
constexpr long long kWaitCycles = 1ll << 31;   // about a second of SM clocks

// Dynamic shared memory, from a 1024-byte aligned base.
struct Smem {
  static constexpr int kA = 0;
  static constexpr int kB = kA + kAbStages * kTileBytes;
  static constexpr int kRaw = kB + kAbStages * kTileBytes;
  static constexpr int kBars = kRaw + kRawStages * kRawBytes;
  // raw_full[3], raw_empty[3], ab_full[4], ab_empty[4], acc_full
  static constexpr int kBarCount = 2 * kRawStages + 2 * kAbStages + 1;
  static constexpr int kTmemSlot = kBars + kBarCount * 8;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kBytes = kAbort + 4 + 1024;   // + room to align the base
};

struct TcGemmArgs {
  const uint8_t* w;        // first row
  int rows;
  int row_bytes;
  int blocks;              // Q4_K blocks per row
  int blocks_per_unit;     // K range of one thread block
  int ksplit;
  const uint8_t* xh;       // activation tile images [blocks * 4][npad][64] fp16, swizzled
  const float* unscale;    // [npad]: factor that undoes the row's power-of-two scale
  int npad;                // tokens rounded up to a multiple of 16
  int tokens;
  float* out;              // ksplit == 1: y + offset; else partial sums [ksplit][tokens][rows]
  int out_stride;          // floats between token rows of out
  size_t split_stride;     // floats between the K ranges' partial sums
  int* error;              // device int: 0, or the code of the first wait that ran out
};

__device__ __forceinline__ uint32_t SharedAddress(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

// Waits for the phase with `parity` to complete, for at most kWaitCycles and
// only while no thread of the block has given up. Returns false when it did
// not see the phase complete.
__device__ __forceinline__ bool BoundedWait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            int* error, int code) {
  if (MbarTryWait(bar, parity)) {
    return true;
  }
  const long long start = clock64();
  while (clock64() - start < kWaitCycles) {
    if (MbarTryWait(bar, parity)) {
      return true;
    }
    if (*abort_flag != 0) {
      return false;
    }
  }
  *abort_flag = 1;
  atomicCAS(error, 0, code);
  return false;
}

__device__ __forceinline__ void BulkCopy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and the
// 128-byte swizzle: start address and offsets in 16-byte units, 1024 bytes
// between 8-row groups, descriptor version 1.
__device__ __forceinline__ uint64_t TileDescriptor(uint32_t shared_address) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((shared_address & 0x3FFFFu) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;           // leading byte offset (unused with swizzle)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;   // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;           // version
  desc |= static_cast<uint64_t>(2) << 61;           // 128-byte swizzle
  return desc;
}

__device__ __forceinline__ void MmaF16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0) : "memory");
}

__device__ __forceinline__ void MmaCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void TmemLoad16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = __uint_as_float(r[i]);
  }
}

// Eight weights of one sub-block from the low nibbles of two words, as four
// fp16 pairs: w = scale * q - offset.
__device__ __forceinline__ uint4 EightWeights(uint32_t w0, uint32_t w1, float scale, float offset) {
  const float q0 = SmallByteToFloat<0>(w0), q1 = SmallByteToFloat<1>(w0);
  const float q2 = SmallByteToFloat<2>(w0), q3 = SmallByteToFloat<3>(w0);
  const float q4 = SmallByteToFloat<0>(w1), q5 = SmallByteToFloat<1>(w1);
  const float q6 = SmallByteToFloat<2>(w1), q7 = SmallByteToFloat<3>(w1);
  const __half2 h0 = __floats2half2_rn(fmaf(q0, scale, -offset), fmaf(q1, scale, -offset));
  const __half2 h1 = __floats2half2_rn(fmaf(q2, scale, -offset), fmaf(q3, scale, -offset));
  const __half2 h2 = __floats2half2_rn(fmaf(q4, scale, -offset), fmaf(q5, scale, -offset));
  const __half2 h3 = __floats2half2_rn(fmaf(q6, scale, -offset), fmaf(q7, scale, -offset));
  return make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                    *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
}

__global__ void __launch_bounds__(kTcThreads, 1)
GemmQ4KTc(const __grid_constant__ TcGemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // The swizzled tiles need a 1024-byte aligned base.
  const uint32_t base = (SharedAddress(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - SharedAddress(smem_raw));
  const uint32_t bars = base + Smem::kBars;
  auto raw_full = [&](int s) { return bars + 8u * s; };
  auto raw_empty = [&](int s) { return bars + 8u * (kRawStages + s); };
  auto ab_full = [&](int s) { return bars + 8u * (2 * kRawStages + s); };
  auto ab_empty = [&](int s) { return bars + 8u * (2 * kRawStages + kAbStages + s); };
  const uint32_t acc_full = bars + 8u * (2 * kRawStages + 2 * kAbStages);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Smem::kTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::kAbort);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile = static_cast<int>(blockIdx.x) / a.ksplit;
  const int split = static_cast<int>(blockIdx.x) % a.ksplit;
  const int first_block = split * a.blocks_per_unit;
  const int unit_blocks = min(a.blocks_per_unit, a.blocks - first_block);   // >= 1 by construction
  const int row0 = tile * kTileRows;
  const uint32_t b_tile_bytes = static_cast<uint32_t>(a.npad) * (kTileK * 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      MbarInit(raw_full(s), 1);
      MbarInit(raw_empty(s), kDequantThreads);
    }
    for (int s = 0; s < kAbStages; ++s) {
      MbarInit(ab_full(s), kDequantThreads + 1);
      MbarInit(ab_empty(s), 1);
    }
    MbarInit(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(base + Smem::kTmemSlot), "r"(kTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  // The weights never depend on earlier kernels; the activation tiles do.
  GridLaunchDependents();

  if (warp == 4) {
    // ---- loader ----------------------------------------------------------
    // Weight blocks are requested kRawStages blocks ahead of the activation
    // tiles, whose buffers only free up as the MMAs retire.
    int raw_next = 0;
    auto request_blocks = [&](int upto) {
      for (; raw_next < upto && raw_next < unit_blocks; ++raw_next) {
        const int s = raw_next % kRawStages;
        const uint32_t phase = (raw_next / kRawStages) & 1u;
        BoundedWait(raw_empty(s), phase ^ 1u, abort_flag, a.error, 1);
        if (lane == 0) {
          MbarArriveExpectTx(raw_full(s), kRawBytes);
        }
        __syncwarp();
        const int block = first_block + raw_next;
#pragma unroll
        for (int rr = 0; rr < kTileRows / 32; ++rr) {
          const int r = rr * 32 + lane;
          // Rows past the end repeat the last row; their sums are never stored.
          const int row = min(row0 + r, a.rows - 1);
          BulkCopy(base + Smem::kRaw + s * kRawBytes + r * kQ4KBytes,
                   a.w + static_cast<size_t>(row) * a.row_bytes + static_cast<size_t>(block) * kQ4KBytes,
                   kQ4KBytes, raw_full(s));
        }
      }
    };
    request_blocks(kRawStages - 1);
    GridDependencyWait();
    int ab_stage = 0;
    uint32_t ab_phase = 0;
    for (int i = 0; i < unit_blocks; ++i) {
      request_blocks(i + kRawStages);
      const int block = first_block + i;
      for (int t = 0; t < 4; ++t) {
        BoundedWait(ab_empty(ab_stage), ab_phase ^ 1u, abort_flag, a.error, 2);
        if (lane == 0) {
          MbarArriveExpectTx(ab_full(ab_stage), b_tile_bytes);
          BulkCopy(base + Smem::kB + ab_stage * kTileBytes,
                   a.xh + (static_cast<size_t>(block) * 4 + t) * b_tile_bytes, b_tile_bytes, ab_full(ab_stage));
        }
        if (++ab_stage == kAbStages) {
          ab_stage = 0;
          ab_phase ^= 1u;
        }
      }
    }
  } else if (warp == 5) {
    // ---- MMA issue ---------------------------------------------------------
    // kind::f16, fp32 accumulate, fp16 A and B, both K-major, N = npad, M = 128.
    const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(a.npad >> 3) << 17) | (8u << 24);
    int ab_stage = 0;
    uint32_t ab_phase = 0;
    for (int i = 0; i < unit_blocks * 4; ++i) {
      BoundedWait(ab_full(ab_stage), ab_phase, abort_flag, a.error, 3);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        const uint64_t desc_a = TileDescriptor(base + Smem::kA + ab_stage * kTileBytes);
        const uint64_t desc_b = TileDescriptor(base + Smem::kB + ab_stage * kTileBytes);
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k) {
          // 16 values = 32 bytes further along K inside the swizzled rows.
          MmaF16(tmem, desc_a + 2u * k, desc_b + 2u * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        MmaCommit(ab_empty(ab_stage));
        if (i == unit_blocks * 4 - 1) {
          MmaCommit(acc_full);
        }
      }
      __syncwarp();
      if (++ab_stage == kAbStages) {
        ab_stage = 0;
        ab_phase ^= 1u;
      }
    }
  } else {
    // ---- dequant: thread r owns weight row r of the tile ---------------------
    const int r = threadIdx.x;
    int ab_stage = 0;
    uint32_t ab_phase = 0;
    for (int i = 0; i < unit_blocks; ++i) {
      const int s = i % kRawStages;
      const uint32_t phase = (i / kRawStages) & 1u;
      BoundedWait(raw_full(s), phase, abort_flag, a.error, 4);
      const uint8_t* block = smem + Smem::kRaw + s * kRawBytes + r * kQ4KBytes;
      const uint4 head = *reinterpret_cast<const uint4*>(block);
      const float d = HalfBitsToFloat(static_cast<uint16_t>(head.x & 0xFFFF));
      const float dmin = HalfBitsToFloat(static_cast<uint16_t>(head.x >> 16));
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        int sc_lo, m_lo, sc_hi, m_hi;
        ScaleMinK4(2 * t, head.y, head.z, head.w, &sc_lo, &m_lo);
        ScaleMinK4(2 * t + 1, head.y, head.z, head.w, &sc_hi, &m_hi);
        const float a_lo = d * static_cast<float>(sc_lo), b_lo = dmin * static_cast<float>(m_lo);
        const float a_hi = d * static_cast<float>(sc_hi), b_hi = dmin * static_cast<float>(m_hi);
        const uint4 q0 = *reinterpret_cast<const uint4*>(block + 16 + 32 * t);
        const uint4 q1 = *reinterpret_cast<const uint4*>(block + 32 + 32 * t);
        const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        BoundedWait(ab_empty(ab_stage), ab_phase ^ 1u, abort_flag, a.error, 5);
        uint8_t* tile_row = smem + Smem::kA + ab_stage * kTileBytes + r * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          // Chunk c: values 8c .. 8c + 7 of the low sub-block; chunk 4 + c: of the high one.
          const uint32_t w0 = words[2 * c], w1 = words[2 * c + 1];
          const uint4 low = EightWeights(w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, a_lo, b_lo);
          const uint4 high = EightWeights((w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu, a_hi, b_hi);
          *reinterpret_cast<uint4*>(tile_row + ((c ^ (r & 7)) << 4)) = low;
          *reinterpret_cast<uint4*>(tile_row + (((4 + c) ^ (r & 7)) << 4)) = high;
        }
        // Make the generic-proxy stores visible to the tensor core's reads.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        MbarArrive(ab_full(ab_stage));
        if (++ab_stage == kAbStages) {
          ab_stage = 0;
          ab_phase ^= 1u;
        }
      }
      MbarArrive(raw_empty(s));
    }
    // ---- epilogue: lane = weight row, column = token ---------------------------
    const bool ready = BoundedWait(acc_full, 0, abort_flag, a.error, 6);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = row0 + r;
    float* out = a.out + static_cast<size_t>(split) * a.split_stride + row;
    for (int col0 = 0; col0 < a.npad; col0 += 16) {
      float v[16];
      TmemLoad16(tmem + (static_cast<uint32_t>(warp * 32) << 16) + col0, v);
      if (ready && row < a.rows) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (col0 + j < a.tokens) {
            out[static_cast<size_t>(col0 + j) * a.out_stride] = v[j] * a.unscale[col0 + j];
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
  }
}

// One block per token row: scales the row by a power of two so that its largest
// magnitude lands in [2^13, 2^14), rounds to fp16 and writes the row into every
// tile image at its swizzled place. Rows past `tokens` are zero.
__global__ void __launch_bounds__(256)
StageHalfKernel(const float* __restrict__ x, int tokens, int cols, int npad, uint8_t* __restrict__ xh,
                float* __restrict__ unscale) {
  __shared__ uint32_t warp_top[8];
  GridDependencyWait();
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  float up = 1.0f;
  if (n < tokens) {
    uint32_t top = 0;
    for (int i = threadIdx.x; i < cols; i += 256) {
      top = max(top, __float_as_uint(x[static_cast<size_t>(n) * cols + i]) & 0x7FFFFFFFu);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      top = max(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
    }
    if (lane == 0) {
      warp_top[warp] = top;
    }
    __syncthreads();
    top = warp_top[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) {
      top = max(top, warp_top[w]);
    }
    // Biased exponent e of the maximum: |x| < 2^(e - 126). Scale by 2^(140 - e)
    // (clamped to normal factors) so the maximum is below 2^14; inf and NaN
    // rows keep factor 1 and stay inf / NaN in fp16.
    int e = static_cast<int>(top >> 23);
    int shift = e == 255 ? 0 : 140 - e;
    shift = max(-126, min(126, shift));
    up = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);
    if (threadIdx.x == 0) {
      unscale[n] = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
    }
  } else if (threadIdx.x == 0) {
    unscale[n] = 0.f;
  }
  const size_t tile_bytes = static_cast<size_t>(npad) * (kTileK * 2);
  for (int chunk = threadIdx.x; chunk < cols / 8; chunk += 256) {
    const int k = chunk * 8;
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    if (n < tokens) {
      const float4 v0 = *reinterpret_cast<const float4*>(x + static_cast<size_t>(n) * cols + k);
      const float4 v1 = *reinterpret_cast<const float4*>(x + static_cast<size_t>(n) * cols + k + 4);
      const __half2 h0 = __floats2half2_rn(v0.x * up, v0.y * up), h1 = __floats2half2_rn(v0.z * up, v0.w * up);
      const __half2 h2 = __floats2half2_rn(v1.x * up, v1.y * up), h3 = __floats2half2_rn(v1.z * up, v1.w * up);
      packed = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                          *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
    }
    const int tile = k / kTileK;
    const int c = (k % kTileK) / 8;
    *reinterpret_cast<uint4*>(xh + tile * tile_bytes + static_cast<size_t>(n) * 128 + ((c ^ (n & 7)) << 4)) = packed;
  }
}

// y[t][row] = sum over the K ranges, in order, of their partial sums.
__global__ void __launch_bounds__(256)
SumSplitsKernel(const float* __restrict__ partial, int ksplit, size_t split_stride, int rows, int tokens,
                float* __restrict__ y, int y_stride) {
  GridDependencyWait();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  const int t = blockIdx.y;
  if (row >= rows || t >= tokens) {
    return;
  }
  float total = 0.f;
  for (int s = 0; s < ksplit; ++s) {
    total += partial[static_cast<size_t>(s) * split_stride + static_cast<size_t>(t) * rows + row];
  }
  y[static_cast<size_t>(t) * y_stride + row] = total;
}

int ReserveTc(gufo_cuda_ctx* ctx, size_t bytes) {
  if (ctx->tc_scratch_bytes >= bytes) {
    return GUFO_CUDA_OK;
  }
  if (ctx->tc_scratch != nullptr) {
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    GUFO_CUDA_TRY(cudaFree(ctx->tc_scratch));
    ctx->tc_scratch = nullptr;
    ctx->tc_scratch_bytes = 0;
  }
  GUFO_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&ctx->tc_scratch), bytes));
  GUFO_CUDA_TRY(cudaMemsetAsync(ctx->tc_scratch, 0, 256, ctx->stream));
  ctx->tc_scratch_bytes = bytes;
  return GUFO_CUDA_OK;
}

}  // namespace

bool TcGemmRuns(const gufo_cuda_ctx* ctx, int type, int cols, int tokens) {
  return !ctx->force_general && ctx->tc_gemm && type == GUFO_CUDA_Q4_K && cols % kSuperBlock == 0 &&
         tokens >= kTcMinTokens;
}

// Scratch layout: [0, 256) error word; then the tile images, the unscale
// factors, and the partial sums of a split product.
int LaunchGemmTc(gufo_cuda_ctx* ctx, const GemvArgs& base, int tokens) {
  const int cols = base.cols;
  const int blocks = cols / kSuperBlock;
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    GUFO_CUDA_TRY(cudaFuncSetAttribute(GemmQ4KTc, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes));
    configured[ctx->device & 15] = true;
  }
  for (int t0 = 0; t0 < tokens; t0 += kTcMaxTokens) {
    const int m = tokens - t0 < kTcMaxTokens ? tokens - t0 : kTcMaxTokens;
    const int npad = (m + 15) / 16 * 16;
    const size_t image_bytes = static_cast<size_t>(blocks) * 4 * npad * (kTileK * 2);
    int max_rows = 0;
    for (int p = 0; p < base.nparts; ++p) {
      max_rows = base.parts[p].rows > max_rows ? base.parts[p].rows : max_rows;
    }
    // Enough thread blocks to cover the SMs once: split K when the rows alone do not.
    auto splits_for = [&](int rows) {
      const int tiles = (rows + kTileRows - 1) / kTileRows;
      int ksplit = 1;
      if (tiles * 5 < ctx->sm_count * 3) {
        ksplit = ctx->sm_count / tiles;
        ksplit = ksplit > blocks ? blocks : ksplit;
        ksplit = ksplit < 1 ? 1 : ksplit;
      }
      const int per = (blocks + ksplit - 1) / ksplit;
      return (blocks + per - 1) / per;   // no empty K range
    };
    size_t partial_floats = 0;
    for (int p = 0; p < base.nparts; ++p) {
      const int ksplit = splits_for(base.parts[p].rows);
      if (ksplit > 1) {
        const size_t need = static_cast<size_t>(ksplit) * m * base.parts[p].rows;
        partial_floats = need > partial_floats ? need : partial_floats;
      }
    }
    const size_t images_at = 256;
    const size_t unscale_at = images_at + (image_bytes + 255) / 256 * 256;
    const size_t partial_at = unscale_at + 1024;
    const int rc = ReserveTc(ctx, partial_at + partial_floats * 4);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
    uint8_t* xh = ctx->tc_scratch + images_at;
    float* unscale = reinterpret_cast<float*>(ctx->tc_scratch + unscale_at);
    float* partial = reinterpret_cast<float*>(ctx->tc_scratch + partial_at);
    const float* x = base.x + static_cast<size_t>(t0) * cols;
    GUFO_CUDA_TRY(LaunchOverlapped(StageHalfKernel, dim3(npad), dim3(256), 0, ctx->stream, 1, x, m, cols, npad, xh,
                                   unscale));
    ctx->launches.fetch_add(1);
    for (int p = 0; p < base.nparts; ++p) {
      const GemvPart& part = base.parts[p];
      TcGemmArgs args{};
      args.w = part.data;
      args.rows = part.rows;
      args.row_bytes = part.row_bytes;
      args.blocks = blocks;
      args.ksplit = splits_for(part.rows);
      args.blocks_per_unit = (blocks + args.ksplit - 1) / args.ksplit;
      args.xh = xh;
      args.unscale = unscale;
      args.npad = npad;
      args.tokens = m;
      args.error = reinterpret_cast<int*>(ctx->tc_scratch);
      float* y = base.y + static_cast<size_t>(t0) * base.y_stride + part.out_offset;
      if (args.ksplit == 1) {
        args.out = y;
        args.out_stride = base.y_stride;
        args.split_stride = 0;
      } else {
        args.out = partial;
        args.out_stride = part.rows;
        args.split_stride = static_cast<size_t>(m) * part.rows;
      }
      const int tiles = (part.rows + kTileRows - 1) / kTileRows;
      GUFO_CUDA_TRY(LaunchOverlapped(GemmQ4KTc, dim3(tiles * args.ksplit), dim3(kTcThreads), Smem::kBytes,
                                     ctx->stream, 1, args));
      ctx->launches.fetch_add(1);
      if (args.ksplit > 1) {
        GUFO_CUDA_TRY(LaunchOverlapped(SumSplitsKernel, dim3((part.rows + 255) / 256, m), dim3(256), 0, ctx->stream, 1,
                                       static_cast<const float*>(partial), args.ksplit, args.split_stride, part.rows,
                                       m, y, base.y_stride));
        ctx->launches.fetch_add(1);
      }
    }
  }
  return GUFO_CUDA_OK;
}

int TcGemmError(gufo_cuda_ctx* ctx, int* code) {
  *code = 0;
  if (ctx->tc_scratch == nullptr) {
    return GUFO_CUDA_OK;
  }
  GUFO_CUDA_TRY(cudaMemcpyAsync(code, ctx->tc_scratch, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  return GUFO_CUDA_OK;
}

}  // namespace gufo
