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

#include "q6k_unit.cuh"

namespace gufo {
namespace {

using namespace q6k;

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
