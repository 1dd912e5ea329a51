// Q4_K GEMV / small-M GEMM on the int8 tensor-core path (see mma_common.cuh for
// the arithmetic). The product is the reference's fused Q4_K row dot
// (gguf_dot::DotK4, src/models/qwen35/gguf_dot.hpp:115-188):
//   y_r = sum_blocks [ d * sum_j sc_j (q_j . x_j)  -  dmin * sum_j m_j (sum x_j) ]
// with the code dots (q_j . x_j) taken exactly by the MMA.
//
// Work split. A persistent grid (a few thread blocks per SM) takes the 16-row
// tiles blockIdx.x, blockIdx.x + gridDim.x, ... A tile is cut into slabs of up
// to eight 256-value blocks; a slab (16 rows x <= 1152 bytes) is copied from
// global to shared memory by the whole thread block with 16-byte asynchronous
// copies, each warp instruction covering 512 contiguous bytes of one row, three
// slabs in flight per thread block. Warp w multiplies block w of the slab from
// shared memory (rows padded by 32 bytes so the 64-bit fragment reads of the
// eight rows of a quarter-warp fall in distinct banks). The warps' partial
// sums for a tile meet in shared memory after the barrier of the next slab.
// The staged activations (three byte planes per token) are copied into shared
// memory once per thread block. The weights never depend on an earlier
// kernel, so the first slabs are requested before the grid-dependency wait.
//
// MMA operand layout (m16n8k32, A row-major u8, B column-major s8). Lane
// (g = lane / 4, t = lane % 4) holds rows g and g + 8. The 32 bytes of a nibble
// pair p carry sub-block 2p in the low and 2p + 1 in the high nibbles; lane t
// loads bytes 8t..8t+7, so its two A words per row are values 8t..8t+3 and
// 8t+4..8t+7 of the sub-block and the matching B words are the same eight
// bytes of column g's plane: one 64-bit shared load, no permutation. High
// nibbles are fed as 16 q (mask 0xF0), the factor 1/16 is folded into the
// column scale.
#include <cooperative_groups.h>

#include "q4k_unit.cuh"

namespace gufo {
namespace {

using namespace q4k;

template <int TOKENS, int PER_SM>
__global__ void __launch_bounds__(kFastThreads, PER_SM)
GemvQ4KMma(const __grid_constant__ FastGemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  // Where the blocks of a cluster leave their sums for block 0: [2][8][16][TOKENS].
  __shared__ float peers[2 * 8 * 16 * TOKENS];
  constexpr int kNB = Accum<TOKENS>::kNB;
  constexpr int kNCols = TOKENS * kLimbs;
  constexpr int kRowFloats = kNCols + TOKENS;   // per row in the exchange buffer
  constexpr int kTileFloats = 16 * kRowFloats;
  const ImageLayout l = MakeImageLayout(TOKENS, a.cols, 32);
  const int blocks = a.cols / kSuperBlock;
  const int slabs_per_tile = (blocks + kSlabBlocks - 1) / kSlabBlocks;
  const float* col_scale = reinterpret_cast<const float*>(smem + l.scale_at);
  const float* sums = reinterpret_cast<const float*>(smem + l.sums_at);
  // After the image: the exchange buffer [2][warps][16 rows][kRowFloats], then
  // the slab ring.
  float* exchange = reinterpret_cast<float*>(smem + l.bytes);
  uint8_t* ring = smem + l.bytes + 2 * kFastWarps * kTileFloats * 4;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  // Column g of the first MMA column group; lanes past the last token's planes
  // wrap onto live ones (see MultiplyPair).
  const uint8_t* lane_plane = smem + (g % kNCols) * l.plane_stride + 8 * t;
  const int tiles_per_group = TotalTiles(a);
  const bool grouped = a.group_ids != nullptr;
  const int row_tiles = grouped ? tiles_per_group * a.groups : tiles_per_group;
  // With ksplit > 1 a cluster of ksplit blocks shares each tile.
  const int ks = a.ksplit > 1 ? a.ksplit : 1;
  const int rank = static_cast<int>(blockIdx.x) % ks;
  const int slot = static_cast<int>(blockIdx.x) / ks;
  const int stride = static_cast<int>(gridDim.x) / ks;
  const int my_tiles = (row_tiles - slot + stride - 1) / stride;
  const int slabs_mine = (slabs_per_tile - rank + ks - 1) / ks;
  const int my_slabs = my_tiles * slabs_mine;
  // A grouped launch has one block per tile; the block's group picks the
  // matrix of each part, the input and the output.
  int group = 0;
  size_t matrix = 0;
  if (grouped) {
    GridDependencyWait();   // the ids come from an earlier kernel
    group = slot / tiles_per_group;
    const int id = a.group_ids[group];
    if (id < 0) {
      return;
    }
    matrix = static_cast<size_t>(id);
  }
  auto locate = [&](int n, int* part, int* local) {
    LocateTile(a, grouped ? slot - group * tiles_per_group : slot + n * stride, part, local);
  };

  // Requests slab q (tile q / slabs_per_tile): warp w copies rows 2w and 2w + 1,
  // a lane the 16-byte chunks lane, lane + 32, lane + 64 of the row's segment.
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
      const int nblk = min(kSlabBlocks, blocks - s * kSlabBlocks);
      const int chunks = nblk * (kQ4KBytes / 16);
      const uint32_t dst0 = ring_base + (q % kStages) * kSlabBytes;
      int part, local;
      locate(n, &part, &local);
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int r = 2 * warp + rr;
        // Rows past the end repeat the last row; their sums are never stored.
        const int row = min(local * 16 + r, a.parts[part].rows - 1);
        const uint8_t* src = a.parts[part].w +
                             (matrix * a.parts[part].rows + static_cast<size_t>(row)) * a.row_bytes +
                             s * (kSlabBlocks * kQ4KBytes);
        const uint32_t dst = dst0 + r * kSlabRowBytes;
#pragma unroll
        for (int c = 0; c < 3; ++c) {
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
    FillImage<TOKENS>(a, l, smem, 1.0f / 16.0f, a.x + static_cast<size_t>(group / (a.x_group_div > 1 ? a.x_group_div : 1)) * a.x_group_stride, rank, ks, kSlabBlocks);
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
    locate(n, &part, &local);
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
      a.y[static_cast<size_t>(group) * a.y_group_stride + static_cast<size_t>(k) * a.y_stride +
          a.parts[part].y_offset + row] = total;
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
      Q4KUnit unit;
      LoadUnit(unit, ring + (q % kStages) * kSlabBytes, warp, g, t);
      MultiplyUnit<TOKENS>(unit, b, g, t, lane_plane, l, col_scale, sums, acc);
    }
    if (s == slabs_mine - 1) {
      // Hand this tile's partial sums to the block.
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
  const ImageLayout l = MakeImageLayout(TOKENS, cols, 32);
  return static_cast<size_t>(l.bytes) +
         static_cast<size_t>(2) * kFastWarps * 16 * (TOKENS * kLimbs + TOKENS) * 4 +
         static_cast<size_t>(kStages) * kSlabBytes;
}

template <int TOKENS, int PER_SM>
int LaunchVariant(gufo_cuda_ctx* ctx, const FastGemvArgs& args) {
  const size_t smem = SharedBytes<TOKENS>(args.cols);
  if (smem > static_cast<size_t>(kFastMaxShared)) {
    return GUFO_CUDA_TOO_LARGE;
  }
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    GUFO_CUDA_TRY(cudaFuncSetAttribute(GemvQ4KMma<TOKENS, PER_SM>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kFastMaxShared));
    configured[ctx->device & 15] = true;
  }
  int row_tiles = 0;
  for (int p = 0; p < args.nparts; ++p) {
    row_tiles += (args.parts[p].rows + 15) / 16;
  }
  // Few rows and several slabs per tile: split the tiles' slabs over a cluster.
  FastGemvArgs launch = args;
  launch.variant = ctx->gemv_variant;
  const int slabs = (args.cols / kSuperBlock + kSlabBlocks - 1) / kSlabBlocks;
  int grid = 1;
  if (args.group_ids != nullptr) {
    if (args.groups <= 0 || args.tokens != 1 || args.prologue == kPrologueImage) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "fast gemv: a grouped launch takes one token and a fused input");
    }
    launch.ksplit = 1;
    grid = row_tiles * args.groups;   // one block per tile
  } else {
    PlanFastGrid(GemvQ4KMma<TOKENS, PER_SM>, ctx->device, kFastThreads, smem, row_tiles, slabs, &launch.ksplit, &grid);
  }
  GUFO_CUDA_TRY(LaunchOverlapped(GemvQ4KMma<TOKENS, PER_SM>, dim3(grid), dim3(kFastThreads), smem,
                                 ctx->stream, launch.ksplit, launch));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

template <int TOKENS>
int Launch(gufo_cuda_ctx* ctx, const FastGemvArgs& args) {
  // One token needs few enough registers for three resident blocks per SM.
  return LaunchVariant<TOKENS, (TOKENS == 1 ? 3 : 2)>(ctx, args);
}

}  // namespace

// Whether `tokens` rows of `cols` values fit the shared-memory image.
bool Q4KFastFits(int cols, int tokens) {
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

// Enqueues one Q4_K part against the staged image `args.image`.
int LaunchGemvQ4KFast(gufo_cuda_ctx* ctx, const FastGemvArgs& args) {
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
