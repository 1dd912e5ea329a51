// Dequant-fused small-M GEMM on the fifth-generation tensor cores: the product
// behind Projections::Apply (GgufProjections::MatMul,
// src/models/qwen35/gguf_projections.cpp:239-286 in the reference) when 16 to
// 128 token rows share one weight read - the ragged verify batch, where every
// sequence brings a few draft tokens and the packed rows form one matrix.
//
// One thread block multiplies 256 weight rows by all the tokens over a range
// of K:
//   D[128 token rows][256 weight rows] (fp32, tensor memory) += X[128][64] * W[256][64]^T
// per 64 columns. The tokens sit on the MMA's M (the tensor core spends M cycles
// per instruction whatever N is, measured here: 128 x 32 x 16 took as long as
// 128 x 128 x 16), the weight rows fill its N = 256.
//   - six loader warps copy one block of each of the 256 rows per stage (Q4_K:
//     its 144 bytes; Q6_K: 208 bytes from the three planes of the device
//     arrangement plus the slab's d values) with 16-byte cp.async whose
//     completion arrives on an mbarrier (tiled TMA boxes this narrow, 144 B wide,
//     ran no faster);
//   - one loader thread brings the activation tiles with one bulk copy
//     (cp.async.bulk) each: the activations were converted once per product into
//     fp16 tile images that already carry the shared-memory swizzle;
//   - sixteen dequant warps, two threads per weight row: w = d*sc*q - dmin*m
//     (DequantQ4_K, src/core/quant.cpp:33-59) in packed fp16 arithmetic (two
//     weights per instruction, as d*sc*(q - 8) + (8*d*sc - dmin*m)) or
//     w = d*sc*(q - 32) (DequantQ6_K, :98-125), likewise two per instruction,
//     stored in the 128-byte-swizzled K-major layout the MMA reads; all sixteen
//     warps work on one tile at a time, in the order the MMA consumes them;
//   - one thread issues tcgen05.mma (kind::f16, M = 128, N = 256, K = 16, four
//     per tile) and tcgen05.commit hands the tile buffers back;
//   - four epilogue warps read the accumulator with tcgen05.ld (lane = token,
//     column = weight row) and store y[token][row] while the other warps are
//     already on the next unit of work: thread blocks are persistent, walk their
//     (row tile, K range) units round-robin, and tensor memory holds two
//     accumulators.
// Each activation row is scaled by a power of two into fp16 range first and the
// outputs scaled back, so range never costs precision. Rounding w and x to
// fp16 (11 significant bits) bounds the relative L2 error of y near 2e-4.
//
// Roofline: weights stream once from HBM (0.5625 B per weight); a tile costs
// 4 MMAs of 128 cycles for 256 x 64 weights, 32 weights per cycle per SM, and
// about 4 instructions per weight of dequant arithmetic. What binds today is
// shared-memory bandwidth: every weight is written as fp16 (2 B) and read by
// the MMA (2 B), its Q4_K bytes pass through shared memory (1.1 B), and the
// activation tile of 16 KiB is written and read once per 16384 weights (2 B):
// about 7 B per weight against 128 B per cycle, 16 to 18 weights per cycle per
// SM, which is what the kernel measures. Matrices with few row tiles split K
// over thread blocks when the modelled time says so; the partial sums are
// added in a fixed order by a second kernel.
//
// Every wait on an mbarrier is bounded: a wait that runs out records an error
// code, raises a block-wide abort flag that ends all other waits, and the
// kernel still frees its tensor memory and returns.
#include "gemm_tc.cuh"

#include <cuda_fp16.h>

#include <vector>

namespace gufo {

namespace {

constexpr int kTileRows = 256;             // weight rows per thread block (the MMA's N)
constexpr int kTokenRows = 128;            // token rows per tile image (the MMA's M)
constexpr int kTileK = 64;                 // values per tile (one swizzle row of fp16)
constexpr int kWTileBytes = kTileRows * kTileK * 2;    // 32 KiB
constexpr int kXTileBytes = kTokenRows * kTileK * 2;   // 16 KiB
// What differs between the block formats: how one block of a row is copied into
// shared memory (16-byte chunks) and how deep the rings are.
template <int TYPE>
struct Quant;

template <>
struct Quant<GUFO_CUDA_Q4_K> {
  static constexpr int kRowBytes = kQ4KBytes;   // shared memory per row and block
  static constexpr int kWStages = 3, kXStages = 3, kRawStages = 2;
  static constexpr int kLoaders = 3;            // loader warps at work (of kLoaderWarps)
  // Chunk `chunk` of block `block` of a row: the GGUF bytes as they are.
  __device__ static const uint8_t* Source(const uint8_t* row, int blocks, int block, int chunk) {
    (void)blocks;
    return row + static_cast<size_t>(block) * kQ4KBytes + chunk * 16;
  }
};

template <>
struct Quant<GUFO_CUDA_Q6_K> {
  // ql 128 | qh 64 | scales 16 | the 16 bytes that hold the slab's d values | 16
  // unused: rows 240 bytes apart, so that the 16-byte reads of eight consecutive
  // rows fall into different banks (224 put rows r and r + 4 into the same).
  static constexpr int kRowBytes = 240;
  static constexpr int kWStages = 2, kXStages = 2, kRawStages = 2;
  static constexpr int kLoaders = 6;
  // The planar device arrangement (Q6KBlockAt): a slab of n blocks stores
  // ql n x 128 | qh n x 64 | scales n x 16 | d n x 2.
  __device__ static const uint8_t* Source(const uint8_t* row, int blocks, int block, int chunk) {
    const int slab = block / kQ6KSlabBlocks;
    const int j = block - slab * kQ6KSlabBlocks;
    const int left = blocks - slab * kQ6KSlabBlocks;
    const int n = left < kQ6KSlabBlocks ? left : kQ6KSlabBlocks;
    const uint8_t* base = row + static_cast<size_t>(slab) * kQ6KSlabBlocks * kQ6KBytes;
    if (chunk < 8) {
      return base + 128 * j + 16 * chunk;
    }
    if (chunk < 12) {
      return base + 128 * n + 64 * j + 16 * (chunk - 8);
    }
    if (chunk == 12) {
      return base + 192 * n + 16 * j;
    }
    return base + 208 * n;   // all of the slab's d values; the row stride covers the 16 bytes
  }
};
constexpr int kDequantThreads = 2 * kTileRows;         // two threads per weight row
constexpr int kEpilogueWarp = kDequantThreads / 32;    // four epilogue warps, one per lane quarter
constexpr int kEpilogueWarps = 4;
constexpr int kLoaderWarp = kEpilogueWarp + kEpilogueWarps;   // and the next: weight loaders
// Up to six of them (Quant<TYPE>::kLoaders at work): with two, in-kernel cycle
// counters showed the loaders issuing copies 70 % (Q4_K) and 98 % (Q6_K) of the
// time while every other role waited.
constexpr int kLoaderWarps = 6;
constexpr int kMmaWarp = kLoaderWarp + kLoaderWarps;
constexpr int kTileLoaderWarp = kMmaWarp + 1;
constexpr int kTcThreads = (kTileLoaderWarp + 1) * 32;
constexpr int kTmemColumns = 512;                      // two accumulators of 256 columns
constexpr long long kWaitCycles = 1ll << 31;   // about a second of SM clocks

// Dynamic shared memory, from a 1024-byte aligned base.
template <int TYPE>
struct Smem {
  using Q = Quant<TYPE>;
  static constexpr int kRawBytes = kTileRows * Q::kRowBytes;   // one block of every row
  static constexpr int kW = 0;
  static constexpr int kX = kW + Q::kWStages * kWTileBytes;
  static constexpr int kRaw = kX + Q::kXStages * kXTileBytes;
  static constexpr int kBars = kRaw + Q::kRawStages * kRawBytes;
  // raw_full, raw_empty, w_full, w_empty, x_full, x_empty (per stage), acc_full[2], acc_empty[2]
  static constexpr int kBarCount = 2 * Q::kRawStages + 2 * Q::kWStages + 2 * Q::kXStages + 4;
  static constexpr int kTmemSlot = kBars + kBarCount * 8;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kBytes = kAbort + 4 + 1024;   // + room to align the base
  static_assert(kX % 1024 == 0 && kRaw % 1024 == 0, "swizzled tiles need 1024-byte alignment");
  static_assert(kBytes <= 227 * 1024, "beyond the shared memory of a thread block");
};

constexpr int kTcMaxParts = 4;

struct TcPart {
  const uint8_t* w;        // first row
  int rows;
  int row_bytes;
  int tiles;               // 256-row tiles of this part
  float* out;              // ksplit == 1: y + offset; else partial sums [ksplit][tokens][rows]
  int out_stride;          // floats between token rows of out
  size_t split_stride;     // floats between the K ranges' partial sums
};

struct TcGemmArgs {
  TcPart parts[kTcMaxParts];
  int nparts;
  int blocks;              // Q4_K blocks per row
  int blocks_per_unit;     // K range of one unit of work
  int ksplit;
  int total_units;         // tiles * ksplit, dealt round-robin to the thread blocks
  int tile_rows;           // weight rows per tile: a multiple of 16 up to kTileRows (the MMA's N)
  const uint8_t* xh;       // activation tile images [blocks * 4][128][64] fp16, swizzled
  const float* unscale;    // [128]: factor that undoes the row's power-of-two scale
  int tokens;
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

// Within every four consecutive values of K the tiles hold them in the order
// (0, 2, 1, 3): a Q4_K word yields the nibbles of its bytes 0 and 2 together (and
// 1 and 3), so this order lets a pair leave the arithmetic as it arrives. The
// activation tiles (StageHalfKernel) and the Q6_K tiles follow the same order;
// a contraction does not care how K is numbered.
//
// Eight weights from two words of a sub-block pair's nibble bytes, in packed
// fp16 arithmetic. A nibble is masked in place under an fp16
// exponent whose mantissa bit there is worth 1 (1024 + code for bits 0-3,
// 64 + code for bits 4-7: one logic instruction for two codes); subtracting the
// power of two plus 8 leaves code - 8 exactly, and one fused multiply-add per
// pair gives w = scale * (code - 8) + (8 * scale - offset). Centring the code
// keeps both terms of the size of w itself, so rounding the scale and the
// constant to fp16 costs about what rounding w does; scale * code - offset
// loses three more bits to cancellation (measured relative L2 of a product:
// 7e-4 that way, 3.8e-4 centred, 2e-4 with fp32 arithmetic rounded once).
__device__ __forceinline__ uint32_t HalfPairFma(uint32_t biased, uint32_t bias, uint32_t scale, uint32_t constant) {
  const __half2 code = __hsub2(*reinterpret_cast<const __half2*>(&biased), *reinterpret_cast<const __half2*>(&bias));
  const __half2 w = __hfma2(code, *reinterpret_cast<const __half2*>(&scale), *reinterpret_cast<const __half2*>(&constant));
  return *reinterpret_cast<const uint32_t*>(&w);
}

// HIGH = false: the low nibbles of the eight bytes of w0 and w1 (eight values of
// sub-block 2t); HIGH = true: the high nibbles (of sub-block 2t + 1).
template <bool HIGH>
__device__ __forceinline__ uint4 EightWeights(uint32_t w0, uint32_t w1, uint32_t scale, uint32_t constant) {
  constexpr uint32_t kMask = HIGH ? 0x00F000F0u : 0x000F000Fu;
  constexpr uint32_t kOne = HIGH ? 0x54005400u : 0x64006400u;    // 64 or 1024 as fp16 pairs
  constexpr uint32_t kBias = HIGH ? 0x54805480u : 0x64086408u;   // 72 or 1032
  const uint32_t s0 = w0 >> 8, s1 = w1 >> 8;
  return make_uint4(HalfPairFma((w0 & kMask) | kOne, kBias, scale, constant),    // bytes 0 and 2
                    HalfPairFma((s0 & kMask) | kOne, kBias, scale, constant),    // bytes 1 and 3
                    HalfPairFma((w1 & kMask) | kOne, kBias, scale, constant),
                    HalfPairFma((s1 & kMask) | kOne, kBias, scale, constant));
}

// Eight Q6_K weights from the codes in the bytes of two words, as four fp16
// pairs, in packed fp16 arithmetic: the codes of bytes 0 and 2 (and 1 and 3) are
// masked in place under the fp16 exponent of 1024, 1024 + 32 is subtracted
// exactly, and one multiply per pair applies the group's scale, itself rounded
// to fp16: w = scale * (code - 32).
__device__ __forceinline__ uint4 EightCodes(uint32_t w0, uint32_t w1, float scale) {
  constexpr uint32_t kMask = 0x003F003Fu, kOne = 0x64006400u, kBias = 0x64206420u;   // 1024, 1056
  const __half2 s2 = __float2half2_rn(scale);
  auto two = [&](uint32_t w) {
    const uint32_t biased = (w & kMask) | kOne;
    const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&biased), *reinterpret_cast<const __half2*>(&kBias)), s2);
    return *reinterpret_cast<const uint32_t*>(&v);
  };
  // Bytes (0, 2) and (1, 3) of each word: the tiles' order of K.
  return make_uint4(two(w0), two(w0 >> 8), two(w1), two(w1 >> 8));
}

// Where unit `u` of a launch works: its part, weight rows and K range.
struct Unit {
  int part;
  int row0;
  int split;
  int first_block;
  int blocks;
};

__device__ __forceinline__ Unit LocateUnit(const TcGemmArgs& a, int u) {
  Unit unit;
  int tile = u / a.ksplit;
  unit.split = u - tile * a.ksplit;
  unit.part = 0;
#pragma unroll
  for (int p = 0; p < kTcMaxParts - 1; ++p) {
    if (unit.part == p && p + 1 < a.nparts && tile >= a.parts[p].tiles) {
      tile -= a.parts[p].tiles;
      unit.part = p + 1;
    }
  }
  unit.row0 = tile * a.tile_rows;
  unit.first_block = unit.split * a.blocks_per_unit;
  unit.blocks = min(a.blocks_per_unit, a.blocks - unit.first_block);   // >= 1 by construction
  return unit;
}

// Row of the MMA's M that token t occupies: tokens are dealt round-robin to the
// four 32-lane quarters of tensor memory, so that all four epilogue warps (each
// can read one quarter) share the work of a small batch.
__host__ __device__ __forceinline__ int TokenRow(int t) { return (t & 3) * 32 + (t >> 2); }

template <int TYPE>
__global__ void __launch_bounds__(kTcThreads, 1)
GemmTc(const __grid_constant__ TcGemmArgs a) {
  using Q = Quant<TYPE>;
  using Smem = Smem<TYPE>;
  constexpr int kWStages = Q::kWStages, kXStages = Q::kXStages, kRawStages = Q::kRawStages;
  constexpr int kRawBytes = Smem::kRawBytes;
  extern __shared__ uint8_t smem_raw[];
  // The swizzled tiles need a 1024-byte aligned base.
  const uint32_t base = (SharedAddress(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - SharedAddress(smem_raw));
  const uint32_t bars = base + Smem::kBars;
  auto raw_full = [&](int s) { return bars + 8u * s; };
  auto raw_empty = [&](int s) { return bars + 8u * (kRawStages + s); };
  auto w_full = [&](int s) { return bars + 8u * (2 * kRawStages + s); };
  auto w_empty = [&](int s) { return bars + 8u * (2 * kRawStages + kWStages + s); };
  auto x_full = [&](int s) { return bars + 8u * (2 * kRawStages + 2 * kWStages + s); };
  auto x_empty = [&](int s) { return bars + 8u * (2 * kRawStages + 2 * kWStages + kXStages + s); };
  auto acc_full = [&](int s) { return bars + 8u * (2 * kRawStages + 2 * kWStages + 2 * kXStages + s); };
  auto acc_empty = [&](int s) { return bars + 8u * (2 * kRawStages + 2 * kWStages + 2 * kXStages + 2 + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Smem::kTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::kAbort);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int units = a.total_units;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      MbarInit(raw_full(s), 32 * Q::kLoaders);
      MbarInit(raw_empty(s), kDequantThreads / 32);
    }
    for (int s = 0; s < kWStages; ++s) {
      MbarInit(w_full(s), kDequantThreads / 32);
      MbarInit(w_empty(s), 1);
    }
    for (int s = 0; s < kXStages; ++s) {
      MbarInit(x_full(s), 1);
      MbarInit(x_empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      MbarInit(acc_full(s), 1);
      MbarInit(acc_empty(s), kEpilogueWarps);
    }
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
  // The weights never depend on earlier kernels; the activation tiles and the
  // outputs do.
  GridLaunchDependents();

  // Every role walks the same units, blockIdx.x, blockIdx.x + gridDim.x, ...;
  // the stage counters run on across units, so the pipeline never drains
  // between them.
  if (warp >= kLoaderWarp && warp < kLoaderWarp + Q::kLoaders) {
    // ---- weight loaders: the 16-byte chunks of one block of every row (Q4_K: 9
    // per row, one 144-byte run; Q6_K: 14 per row from its four planes), split
    // between the loader warps; consecutive lanes take consecutive chunks -------
    const int which = warp - kLoaderWarp;
    constexpr int kChunksPerRow = Q::kRowBytes / 16;
    const int kChunks = a.tile_rows * kChunksPerRow;
    int i = 0;   // blocks requested so far
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const Unit unit = LocateUnit(a, u);
      const TcPart& part = a.parts[unit.part];
      for (int b = 0; b < unit.blocks; ++b, ++i) {
        const int s = i % kRawStages;
        const uint32_t phase = (i / kRawStages) & 1u;
        BoundedWait(raw_empty(s), phase ^ 1u, abort_flag, a.error, 1);
        const uint32_t to = base + Smem::kRaw + s * kRawBytes;
        if constexpr (TYPE == GUFO_CUDA_Q4_K) {
#pragma unroll 6
          for (int c = which * 32 + lane; c < kChunks; c += 32 * Q::kLoaders) {
            const int r = c / kChunksPerRow;
            const int chunk = c - r * kChunksPerRow;
            // Rows past the end repeat the last row; their sums are never stored.
            const int row = min(unit.row0 + r, part.rows - 1);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to + c * 16),
                         "l"(Q::Source(part.w + static_cast<size_t>(row) * part.row_bytes, a.blocks,
                                       unit.first_block + b, chunk)) : "memory");
          }
        } else {
          // Plane by plane (ql: 8 chunks a row, qh: 4, scales: 1, the slab's d values: 1),
          // so that a warp's lanes never part ways over which plane a chunk is in and the
          // offsets of a plane are computed once a block.
          const int block = unit.first_block + b;
          const int slab = block / kQ6KSlabBlocks;
          const int j = block - slab * kQ6KSlabBlocks;
          const int left = a.blocks - slab * kQ6KSlabBlocks;
          const int n = left < kQ6KSlabBlocks ? left : kQ6KSlabBlocks;
          const uint8_t* from = part.w + static_cast<size_t>(slab) * kQ6KSlabBlocks * kQ6KBytes;
          const int last = part.rows - 1 - unit.row0;
          auto plane = [&](int src_at, int dst_at, int shift) {
            // 1 << shift chunks a row.
            const int items = a.tile_rows << shift;
#pragma unroll 4
            for (int c = which * 32 + lane; c < items; c += 32 * Q::kLoaders) {
              const int r = c >> shift;
              const int chunk = c & ((1 << shift) - 1);
              const int row = unit.row0 + min(r, last);
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to + r * Q::kRowBytes + dst_at + 16 * chunk),
                           "l"(from + static_cast<size_t>(row) * part.row_bytes + src_at + 16 * chunk) : "memory");
            }
          };
          plane(128 * j, 0, 3);
          plane(128 * n + 64 * j, 128, 2);
          plane(192 * n + 16 * j, 192, 0);
          plane(208 * n, 208, 0);
        }
        // Arrives on the stage's barrier once this thread's copies have landed.
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(raw_full(s)) : "memory");
      }
    }
  } else if (warp == kTileLoaderWarp) {
    // ---- activation tile loader ------------------------------------------------
    GridDependencyWait();
    int stage = 0;
    uint32_t phase = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const Unit unit = LocateUnit(a, u);
      for (int i = 0; i < unit.blocks * 4; ++i) {
        BoundedWait(x_empty(stage), phase ^ 1u, abort_flag, a.error, 2);
        if (lane == 0) {
          MbarArriveExpectTx(x_full(stage), kXTileBytes);
          BulkCopy(base + Smem::kX + stage * kXTileBytes,
                   a.xh + (static_cast<size_t>(unit.first_block) * 4 + i) * kXTileBytes, kXTileBytes, x_full(stage));
        }
        if (++stage == kXStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ---- MMA issue ---------------------------------------------------------
    // kind::f16, fp32 accumulate, fp16 A and B, both K-major, N = 256, M = 128.
    const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(a.tile_rows >> 3) << 17) |
                           (static_cast<uint32_t>(kTokenRows >> 4) << 24);
    int ws = 0, xs = 0;
    uint32_t w_phase = 0, x_phase = 0;
    int n = 0;   // units done
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++n) {
      const Unit unit = LocateUnit(a, u);
      const int buffer = n & 1;
      // The epilogue of the unit before last has read this accumulator.
      BoundedWait(acc_empty(buffer), ((n >> 1) & 1u) ^ 1u, abort_flag, a.error, 8);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t accumulator = tmem + static_cast<uint32_t>(buffer * kTileRows);
      for (int i = 0; i < unit.blocks * 4; ++i) {
        BoundedWait(w_full(ws), w_phase, abort_flag, a.error, 3);
        BoundedWait(x_full(xs), x_phase, abort_flag, a.error, 7);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (lane == 0) {
          const uint64_t desc_x = TileDescriptor(base + Smem::kX + xs * kXTileBytes);
          const uint64_t desc_w = TileDescriptor(base + Smem::kW + ws * kWTileBytes);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) {
            // 16 values = 32 bytes further along K inside the swizzled rows.
            MmaF16(accumulator, desc_x + 2u * k, desc_w + 2u * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          // Each commit arrives once everything issued so far has retired.
          MmaCommit(w_empty(ws));
          MmaCommit(x_empty(xs));
          if (i == unit.blocks * 4 - 1) {
            MmaCommit(acc_full(buffer));
          }
        }
        __syncwarp();
        if (++ws == kWStages) {
          ws = 0;
          w_phase ^= 1u;
        }
        if (++xs == kXStages) {
          xs = 0;
          x_phase ^= 1u;
        }
      }
    }
  } else if (warp >= kEpilogueWarp && warp < kEpilogueWarp + kEpilogueWarps) {
    // ---- epilogue: lane of tensor memory = token row, column = weight row;
    // warp q reads quarter q, i.e. tokens q, q + 4, q + 8, ... -------------------
    const int quarter = warp - kEpilogueWarp;
    const int token = lane * 4 + quarter;
    int n = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++n) {
      const Unit unit = LocateUnit(a, u);
      const TcPart& part = a.parts[unit.part];
      const int buffer = n & 1;
      const bool ready = BoundedWait(acc_full(buffer), (n >> 1) & 1u, abort_flag, a.error, 6);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool live = ready && token < a.tokens;
      const float unscale = live ? a.unscale[token] : 0.f;
      float* out = part.out + static_cast<size_t>(unit.split) * part.split_stride +
                   static_cast<size_t>(token) * part.out_stride + unit.row0;
      // 16-byte stores where the output rows allow them.
      const bool vector_stores = (reinterpret_cast<uintptr_t>(part.out) & 15) == 0 && part.out_stride % 4 == 0 &&
                                 part.split_stride % 4 == 0;
      // A quarter without tokens is skipped (uniform over the warp, as
      // tcgen05.ld requires).
      if (quarter < a.tokens) {
        for (int col0 = 0; col0 < a.tile_rows; col0 += 16) {
          float v[16];
          TmemLoad16(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * kTileRows + col0, v);
          if (live) {
            if (vector_stores && unit.row0 + col0 + 16 <= part.rows) {
#pragma unroll
              for (int j = 0; j < 16; j += 4) {
                *reinterpret_cast<float4*>(out + col0 + j) =
                    make_float4(v[j] * unscale, v[j + 1] * unscale, v[j + 2] * unscale, v[j + 3] * unscale);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (unit.row0 + col0 + j < part.rows) {
                  out[col0 + j] = v[j] * unscale;
                }
              }
            }
          }
        }
      }
      // This accumulator may be overwritten now.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        MbarArrive(acc_empty(buffer));
      }
    }
  } else if (warp < kDequantThreads / 32) {
    // ---- dequant: threads r and r + 256 own weight row r; all sixteen warps
    // work on the same tile, in the order the MMA consumes them (the first
    // thread takes the first half of each tile row, the second the other).
    // Tile g = 4 * block + t of the thread block's stream lands in buffer g % stages.
    const int r = threadIdx.x & (kTileRows - 1);
    const int half = threadIdx.x / kTileRows;
    const bool active = r < a.tile_rows;   // rows past the tile's height: the barriers only
    int i = 0;   // blocks done so far
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const Unit unit = LocateUnit(a, u);
      for (int b = 0; b < unit.blocks; ++b, ++i) {
        const int s = i % kRawStages;
        const uint32_t phase = (i / kRawStages) & 1u;
        BoundedWait(raw_full(s), phase, abort_flag, a.error, 4);
        if constexpr (TYPE == GUFO_CUDA_Q4_K) {
          const uint8_t* block = smem + Smem::kRaw + s * kRawBytes + r * Q::kRowBytes;
          const uint4 head = *reinterpret_cast<const uint4*>(block);
          const float d = HalfBitsToFloat(static_cast<uint16_t>(head.x & 0xFFFF));
          const float dmin = HalfBitsToFloat(static_cast<uint16_t>(head.x >> 16));
  #pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int g = 4 * i + t;
            const int ws = g % kWStages;
            const uint32_t w_phase = static_cast<uint32_t>(g / kWStages) & 1u;
            // This thread's sub-block of the pair: its scale and the constant
            // 8 * scale - offset, each doubled into an fp16 pair.
            int sc, m;
            ScaleMinK4(2 * t + half, head.y, head.z, head.w, &sc, &m);
            auto pair = [](float v) {
              const __half2 h = __float2half2_rn(v);
              return *reinterpret_cast<const uint32_t*>(&h);
            };
            const float scale = d * static_cast<float>(sc);
            const uint32_t scale2 = pair(scale);
            const uint32_t constant2 = pair(fmaf(8.0f, scale, -dmin * static_cast<float>(m)));
            const uint4 q0 = *reinterpret_cast<const uint4*>(block + 16 + 32 * t);
            const uint4 q1 = *reinterpret_cast<const uint4*>(block + 32 + 32 * t);
            const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            BoundedWait(w_empty(ws), w_phase ^ 1u, abort_flag, a.error, 5);
            uint8_t* tile_row = smem + Smem::kW + ws * kWTileBytes + r * 128;
  #pragma unroll
            for (int c = 0; c < 4; ++c) {
              // Chunk c: values 8c .. 8c + 7 of the low sub-block; chunk 4 + c: of the high one.
              if (active) {
                const uint4 eight = half == 0 ? EightWeights<false>(words[2 * c], words[2 * c + 1], scale2, constant2)
                                              : EightWeights<true>(words[2 * c], words[2 * c + 1], scale2, constant2);
                *reinterpret_cast<uint4*>(tile_row + (((4 * half + c) ^ (r & 7)) << 4)) = eight;
              }
            }
            // Make the generic-proxy stores visible to the tensor core's reads; one
            // lane then arrives for the warp.
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              MbarArrive(w_full(ws));
            }
          }
        } else {
          // Tile t of the block holds values 64t .. 64t + 63: half n = t / 2 of
          // the block, the low (t even) or high nibbles of its 64 ql bytes, two
          // bits of its 32 qh bytes: w = d * sc * (code - 32), code = nibble |
          // two bits of qh << 4 (DequantQ6_K, src/core/quant.cpp:98-125). This
          // thread takes chunks 4 * half .. 4 * half + 3 of every tile: ql bytes
          // 32 * half .. + 31 of the tile's half.
          const uint8_t* block = smem + Smem::kRaw + s * kRawBytes + r * Q::kRowBytes;
          const float d = HalfBitsToFloat(*reinterpret_cast<const uint16_t*>(
              block + 208 + 2 * ((unit.first_block + b) % kQ6KSlabBlocks)));
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            const uint4 l0 = *reinterpret_cast<const uint4*>(block + 64 * n + 32 * half);
            const uint4 l1 = *reinterpret_cast<const uint4*>(block + 64 * n + 32 * half + 16);
            const uint4 h0 = *reinterpret_cast<const uint4*>(block + 128 + 32 * n);
            const uint4 h1 = *reinterpret_cast<const uint4*>(block + 128 + 32 * n + 16);
            const uint2 sc8 = *reinterpret_cast<const uint2*>(block + 192 + 8 * n);
            const uint32_t ql[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
            const uint32_t qh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
            // Scale of 16-value group j of this half of the block (int8).
            auto scale = [&](int j) {
              const uint32_t word = j < 4 ? sc8.x : sc8.y;
              return d * static_cast<float>(static_cast<int>(word << (24 - 8 * (j & 3))) >> 24);
            };
#pragma unroll
            for (int tt = 0; tt < 2; ++tt) {
              const int g = 4 * i + 2 * n + tt;
              const int ws = g % kWStages;
              const uint32_t w_phase = static_cast<uint32_t>(g / kWStages) & 1u;
              BoundedWait(w_empty(ws), w_phase ^ 1u, abort_flag, a.error, 5);
              uint8_t* tile_row = smem + Smem::kW + ws * kWTileBytes + r * 128;
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                // Chunk 4 * half + k: values from ql bytes 32 * half + 8k .., their two
                // high bits from qh bytes 8k .. at bit 2 * (2 tt + half).
                const int shift = 2 * (2 * tt + half);
                const uint32_t q0 = ql[2 * k], q1 = ql[2 * k + 1];
                const uint32_t n0 = tt == 0 ? (q0 & 0x0F0F0F0Fu) : ((q0 >> 4) & 0x0F0F0F0Fu);
                const uint32_t n1 = tt == 0 ? (q1 & 0x0F0F0F0Fu) : ((q1 >> 4) & 0x0F0F0F0Fu);
                const uint32_t b0 = shift <= 4 ? (qh[2 * k] << (4 - shift)) : (qh[2 * k] >> (shift - 4));
                const uint32_t b1 = shift <= 4 ? (qh[2 * k + 1] << (4 - shift)) : (qh[2 * k + 1] >> (shift - 4));
                const float sc = scale(4 * tt + 2 * half + (k >> 1));
                if (active) {
                  *reinterpret_cast<uint4*>(tile_row + (((4 * half + k) ^ (r & 7)) << 4)) =
                      EightCodes(n0 | (b0 & 0x30303030u), n1 | (b1 & 0x30303030u), sc);
                }
              }
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) {
                MbarArrive(w_full(ws));
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) {
          MbarArrive(raw_empty(s));
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
  const int n = blockIdx.x;                  // token
  const int image_row = TokenRow(n);        // its row of the MMA's M
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
      // Values (0, 2, 1, 3) of every four: the order of K the weight tiles use.
      const __half2 h0 = __floats2half2_rn(v0.x * up, v0.z * up), h1 = __floats2half2_rn(v0.y * up, v0.w * up);
      const __half2 h2 = __floats2half2_rn(v1.x * up, v1.z * up), h3 = __floats2half2_rn(v1.y * up, v1.w * up);
      packed = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                          *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
    }
    const int tile = k / kTileK;
    const int c = (k % kTileK) / 8;
    *reinterpret_cast<uint4*>(xh + tile * tile_bytes + static_cast<size_t>(image_row) * 128 +
                              ((c ^ (image_row & 7)) << 4)) = packed;
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
  // An outgrown block is kept (a captured graph may hold it); its error word
  // is not carried over: a failure is read from the current block.
  const int rc = ctx->GrowScratch(&ctx->tc_scratch, &ctx->tc_scratch_bytes, bytes, 1u << 20, "tcgen05 gemm");
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  GUFO_CUDA_TRY(cudaMemsetAsync(ctx->tc_scratch, 0, 256, ctx->stream));
  return GUFO_CUDA_OK;
}


}  // namespace

bool TcGemmRuns(const gufo_cuda_ctx* ctx, int type, int cols, int tokens) {
  if (ctx->force_general || !ctx->tc_gemm || cols % kSuperBlock != 0) {
    return false;
  }
  // "tc_gemm" = 2 sends every product of 16 or more rows here (tests).
  const int least = ctx->tc_gemm_all ? 16 : (type == GUFO_CUDA_Q6_K ? kTcMinTokensQ6K : kTcMinTokens);
  return (type == GUFO_CUDA_Q4_K || type == GUFO_CUDA_Q6_K) && tokens >= least;
}

// Scratch layout: [0, 256) error word; then the tile images, the unscale
// factors, and the partial sums of a split product.
int LaunchGemmTc(gufo_cuda_ctx* ctx, const GemvArgs& base, int tokens) {
  const int cols = base.cols;
  const int blocks = cols / kSuperBlock;
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    GUFO_CUDA_TRY(cudaFuncSetAttribute(GemmTc<GUFO_CUDA_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Smem<GUFO_CUDA_Q4_K>::kBytes));
    GUFO_CUDA_TRY(cudaFuncSetAttribute(GemmTc<GUFO_CUDA_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Smem<GUFO_CUDA_Q6_K>::kBytes));
    configured[ctx->device & 15] = true;
  }
  // Launch groups: parts of one block format, up to kTcMaxParts each.
  std::vector<std::vector<int>> groups;
  for (int type : {GUFO_CUDA_Q4_K, GUFO_CUDA_Q6_K}) {
    std::vector<int> group;
    for (int p = 0; p < base.nparts; ++p) {
      if ((reinterpret_cast<uintptr_t>(base.parts[p].data) & 15) != 0 || base.parts[p].row_bytes % 16 != 0) {
        return Fail(GUFO_CUDA_BAD_ARGUMENT, "tcgen05 gemm: weight rows must be 16-byte aligned");
      }
      if (base.parts[p].type != type) {
        continue;
      }
      group.push_back(p);
      if (static_cast<int>(group.size()) == kTcMaxParts) {
        groups.push_back(group);
        group.clear();
      }
    }
    if (!group.empty()) {
      groups.push_back(group);
    }
  }
  // K ranges per 256-row tile; up to kTcMaxParts parts share a launch and its split.
  // The split with the least modelled time: rounds of units over the persistent
  // thread blocks, each a K range plus a little for the accumulator hand-over;
  // a split pays for its partial sums; ties go to the smaller split.
  auto splits_for = [&](int tiles, int m) {
    // In units of one block's time on one SM (about 1.5 us): what the partial
    // sums of one more K range cost in HBM traffic, written once and read once.
    const double range_cost = 2.0 * m * (static_cast<double>(tiles) * kTileRows) * 4.0 / 6.0e6 / 1.5;
    int best = 1;
    double best_cost = 1e30;
    for (int ksplit = 1; ksplit <= blocks; ++ksplit) {
      const int per = (blocks + ksplit - 1) / ksplit;
      const int ranges = (blocks + per - 1) / per;   // no empty K range
      if (ranges != ksplit) {
        continue;
      }
      const int rounds = (tiles * ksplit + ctx->sm_count - 1) / ctx->sm_count;
      const double cost = rounds * (per + 0.3) + (ksplit > 1 ? 2.0 + ksplit * range_cost : 0.0);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best = ksplit;
      }
    }
    return best;
  };
  // Weight rows per tile for a group of parts: the height (a multiple of 16, up
  // to 256) with the least modelled time over the persistent thread blocks. A
  // unit's time falls with its rows until the tensor core's share (it spends as
  // long on a narrow tile as on a wide one) takes over at about half height.
  auto tiles_of = [&](const std::vector<int>& group, int tile_rows) {
    int tiles = 0;
    for (int p : group) {
      tiles += (base.parts[p].rows + tile_rows - 1) / tile_rows;
    }
    return tiles;
  };
  auto tile_rows_for = [&](const std::vector<int>& group) {
    int best = kTileRows;
    double best_cost = 1e30;
    for (int tr = kTileRows; tr >= 64; tr -= 16) {
      const int tiles = tiles_of(group, tr);
      const int rounds = (tiles + ctx->sm_count - 1) / ctx->sm_count;
      const double unit = tr / static_cast<double>(kTileRows);
      const double cost = rounds * (unit > 0.55 ? unit : 0.55);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best = tr;
      }
    }
    return best;
  };
  for (int t0 = 0; t0 < tokens; t0 += kTcMaxTokens) {
    const int m = tokens - t0 < kTcMaxTokens ? tokens - t0 : kTcMaxTokens;
    const size_t image_bytes = static_cast<size_t>(blocks) * 4 * kXTileBytes;
    // Worst case for the partial sums: every part split into blocks / 2 ranges.
    size_t partial_floats = 0;
    for (const std::vector<int>& group : groups) {
      size_t rows = 0;
      for (int p : group) {
        rows += base.parts[p].rows;
      }
      const int tiles = tiles_of(group, tile_rows_for(group));
      const int ksplit = splits_for(tiles, m);
      if (ksplit > 1) {
        const size_t need = static_cast<size_t>(ksplit) * m * rows;
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
    GUFO_CUDA_TRY(LaunchOverlapped(StageHalfKernel, dim3(kTokenRows), dim3(256), 0, ctx->stream, 1, x, m, cols,
                                   kTokenRows, xh, unscale));
    ctx->launches.fetch_add(1);
    for (const std::vector<int>& group : groups) {
      TcGemmArgs args{};
      args.blocks = blocks;
      args.xh = xh;
      args.unscale = unscale;
      args.tokens = m;
      args.error = reinterpret_cast<int*>(ctx->tc_scratch);
      args.tile_rows = tile_rows_for(group);
      const int tiles = tiles_of(group, args.tile_rows);
      args.ksplit = splits_for(tiles, m);
      args.blocks_per_unit = (blocks + args.ksplit - 1) / args.ksplit;
      float* next_partial = partial;
      for (int p : group) {
        const GemvPart& part = base.parts[p];
        TcPart& to = args.parts[args.nparts++];
        to.w = part.data;
        to.rows = part.rows;
        to.row_bytes = part.row_bytes;
        to.tiles = (part.rows + args.tile_rows - 1) / args.tile_rows;
        if (args.ksplit == 1) {
          to.out = base.y + static_cast<size_t>(t0) * base.y_stride + part.out_offset;
          to.out_stride = base.y_stride;
          to.split_stride = 0;
        } else {
          to.out = next_partial;
          to.out_stride = part.rows;
          to.split_stride = static_cast<size_t>(m) * part.rows;
          next_partial += static_cast<size_t>(args.ksplit) * m * part.rows;
        }
      }
      args.total_units = tiles * args.ksplit;
      const int grid = args.total_units < ctx->sm_count ? args.total_units : ctx->sm_count;
      if (base.parts[group[0]].type == GUFO_CUDA_Q4_K) {
        GUFO_CUDA_TRY(LaunchOverlapped(GemmTc<GUFO_CUDA_Q4_K>, dim3(grid), dim3(kTcThreads),
                                       Smem<GUFO_CUDA_Q4_K>::kBytes, ctx->stream, 1, args));
      } else {
        GUFO_CUDA_TRY(LaunchOverlapped(GemmTc<GUFO_CUDA_Q6_K>, dim3(grid), dim3(kTcThreads),
                                       Smem<GUFO_CUDA_Q6_K>::kBytes, ctx->stream, 1, args));
      }
      ctx->launches.fetch_add(1);
      if (args.ksplit > 1) {
        for (int i = 0; i < args.nparts; ++i) {
          const GemvPart& part = base.parts[group[i]];
          float* y = base.y + static_cast<size_t>(t0) * base.y_stride + part.out_offset;
          GUFO_CUDA_TRY(LaunchOverlapped(SumSplitsKernel, dim3((part.rows + 255) / 256, m), dim3(256), 0, ctx->stream,
                                         1, static_cast<const float*>(args.parts[i].out), args.ksplit,
                                         args.parts[i].split_stride, part.rows, m, y, base.y_stride));
          ctx->launches.fetch_add(1);
        }
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


