// Q4_K and Q6_K GEMV / small-M GEMM (1..8 tokens) on the int8 tensor-core
// path: the reference's fused row dots (gguf_dot::DotK4 and DotQ6_K,
// src/models/qwen35/gguf_dot.hpp:115-188,203-290) with the code dots taken
// exactly by mma.sync (arithmetic in mma_common.cuh, the per-unit math and the
// MMA operand layouts in q4k_unit.cuh and q6k_unit.cuh).
//   Q4_K: y_r = sum_blocks [ d * sum_j sc_j (q_j . x_j)  -  dmin * sum_j m_j (sum x_j) ]
//   Q6_K: y_r = sum_blocks d * sum_g sc_g * ((q - 32) . x)_g        g = 16-value groups
//
// Work split. A persistent grid (a few thread blocks per SM) takes the 16-row
// tiles blockIdx.x, blockIdx.x + gridDim.x, ... A tile is cut into slabs of up
// to eight 256-value blocks. A slab (16 rows x <= 1152 or 1680 bytes; Q6_K rows
// in the planar device arrangement of common.cuh) is brought into a ring slot in
// shared memory by sixteen bulk copies (cp.async.bulk, one per row, rows padded
// so that the fragment reads of a quarter-warp fall in distinct banks) that
// complete on the slot's mbarrier; warp w multiplies block w of the slab. The
// weights never depend on an earlier kernel, so the first slabs are requested
// before the grid-dependency wait.
//
// Per slab the eight warps meet once: each waits for the slot's barrier, reads
// its fragments into registers, and after the block's barrier the slot is free
// again, so warp q % 8 requests the slab kStages further on into it (the duty
// rotates) while everyone multiplies. At the end of a tile a warp reduces its
// row sums over its quads and leaves them in one of two exchange buffers;
// after the next slab's barrier sixteen threads per token add the eight warps'
// sums in a fixed order and write y. Launches with few row tiles share a tile's
// slabs over a thread-block cluster: the partial sums cross to the cluster's
// first block through distributed shared memory. (Tried and dropped: no block
// barrier at all, the last warp to release a slot refilling it and the last
// warp to finish a tile adding it up, both through shared-memory counters; it
// ran 20 % slower on the 262144 x 2048 product.)
#include <cooperative_groups.h>

#include <type_traits>

#include "peer.cuh"
#include "q4k_unit.cuh"
#include "q6k_unit.cuh"

namespace gufo {
namespace {

template <int TYPE>
struct Slab;
template <>
struct Slab<GUFO_CUDA_Q4_K> {
  static constexpr int kRowBytes = q4k::kSlabRowBytes;
  static constexpr int kBytes = q4k::kSlabBytes;
  static constexpr int kDataBytes = 8 * kQ4KBytes;   // of a full slab of one row
  static constexpr int kStages = 3;
  static constexpr int kGroup = 32;                   // values per entry of the image's sums
  static constexpr bool kZeros = false;
  static constexpr float kExtra = 1.0f / 16.0f;       // high nibbles reach the MMA as 16 q
};
template <>
struct Slab<GUFO_CUDA_Q6_K> {
  static constexpr int kRowBytes = q6k::kSlabRowBytes;
  static constexpr int kBytes = q6k::kSlabBytes;
  static constexpr int kDataBytes = q6k::kSlabDataBytes;
  static constexpr int kStages = 2;
  static constexpr int kGroup = 16;
  static constexpr bool kZeros = true;                // a plane of zeros behind the image
  static constexpr float kExtra = 0.25f;              // codes reach the MMA as 4 (q - 32)
};

constexpr int kMaxStages = 3;
constexpr int kExchange = 2;

// ONE: every block of the launch multiplies a single slab, so the ring is one
// slot (a third or half of the shared memory: more blocks fit an SM, which lets a
// cluster of three split a three-slab row where two-slot blocks allowed two).
template <int TYPE, int TOKENS, bool ONE = false>
size_t SharedBytes(int cols) {
  const ImageLayout l = MakeImageLayout(TOKENS, cols, Slab<TYPE>::kGroup);
  return static_cast<size_t>(l.bytes) + (Slab<TYPE>::kZeros ? l.plane_stride : 0) +
         static_cast<size_t>(kExchange) * kFastWarps * 16 * TOKENS * 4 +
         static_cast<size_t>(ONE ? 1 : Slab<TYPE>::kStages) * Slab<TYPE>::kBytes;
}

template <int TYPE, int TOKENS, int PER_SM, bool ONE = false>
__global__ void __launch_bounds__(kFastThreads, PER_SM)
GemvMma(const __grid_constant__ FastGemvArgs a) {
  using S = Slab<TYPE>;
  constexpr bool kQ4 = TYPE == GUFO_CUDA_Q4_K;
  constexpr int kStages = ONE ? 1 : S::kStages;
  constexpr int kNCols = TOKENS * kLimbs;
  constexpr int kNB = (kNCols + 7) / 8;
  constexpr int kTileFloats = 16 * TOKENS;   // per warp in an exchange buffer: row sums per token
  extern __shared__ __align__(16) uint8_t smem[];
  // Where the blocks of a cluster leave their sums for block 0: [2][8][16][TOKENS].
  __shared__ float peers[2 * 8 * 16 * TOKENS];
  __shared__ __align__(8) uint64_t landed[kMaxStages];   // a slab's bytes have arrived
  // The barriers need no kernel argument: set up first, while the arguments' first
  // reads (constant-cache misses) are under way. A barrier takes eight arrivals.
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      MbarInit(SharedAddress(&landed[s]), kFastWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  const ImageLayout l = MakeImageLayout(TOKENS, a.cols, S::kGroup);
  const int blocks = a.cols / kSuperBlock;
  const int slabs_per_tile = (blocks + 7) / 8;
  const float* col_scale = reinterpret_cast<const float*>(smem + l.scale_at);
  const float* sums = reinterpret_cast<const float*>(smem + l.sums_at);
  // After the image: (Q6_K) a plane of zeros, the exchange buffers
  // [kExchange][warps][16 rows][TOKENS], then the slab ring.
  uint8_t* zeros = smem + l.bytes;
  float* exchange = reinterpret_cast<float*>(zeros + (S::kZeros ? l.plane_stride : 0));
  uint8_t* ring = reinterpret_cast<uint8_t*>(exchange + kExchange * kFastWarps * kTileFloats);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  // Lane planes of the two unit kinds (q4k_unit.cuh, q6k_unit.cuh): column g of
  // the first MMA column group; lanes past the last token's planes wrap onto
  // live ones, whose sums meet a zero column factor.
  const uint8_t* lane_plane = smem + (g % kNCols) * l.plane_stride + 8 * t;
  const uint8_t* none = zeros + 8 * t;
  const bool one_live = (g & 3) < kNCols && ((g < 4) == (t < 2));
  const uint8_t* lane_first = TOKENS == 1 ? (one_live ? smem + (g & 3) * l.plane_stride + 8 * t : none)
                                          : (t < 2 ? lane_plane : none);
  const uint8_t* lane_second = t < 2 ? none : lane_plane;
  const int tiles_per_group = TotalTiles(a);
  const bool grouped = a.group_ids != nullptr;
  const int row_tiles = grouped ? tiles_per_group * a.groups : tiles_per_group;
  // With ksplit > 1 a cluster of ksplit blocks shares each tile.
  // (No division here: a block's first slabs cannot be requested before these
  // are known, and nothing hides a chain of integer divisions at a kernel's start.
  // A cluster launch has one cluster per tile; the launcher divides the rest.)
  const int ks = a.ksplit > 1 ? a.ksplit : 1;
  int rank = 0;
  int slot = static_cast<int>(blockIdx.x);
  int stride = static_cast<int>(gridDim.x);
  int my_tiles = a.tiles_each + (slot < a.tiles_more ? 1 : 0);
  int slabs_mine = slabs_per_tile;
  if (ks > 1) {
    asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    asm("mov.u32 %0, %%clusterid.x;" : "=r"(slot));
    stride = row_tiles;
    my_tiles = 1;
    slabs_mine = 0;
    for (int s = rank; s < slabs_per_tile; s += ks) {
      ++slabs_mine;
    }
  }
  const int my_slabs = my_tiles * slabs_mine;
  // A grouped launch has one block per tile; the block's group picks the
  // matrix of each part, the input and the output.
  int group = 0;
  size_t matrix = 0;
  // Grouped launches give a block one tile of its group, or (SwiGLU epilogue) one
  // gate tile and the up tile of the same rows.
  const int units_per_group = a.epilogue == kEpilogueSwiGlu ? tiles_per_group / 2 : tiles_per_group;
  if (grouped) {
    GridDependencyWait();   // the ids come from an earlier kernel
    group = slot / units_per_group;
    const int id = a.group_ids[group];
    if (id < 0) {
      return;
    }
    matrix = static_cast<size_t>(id);
  }
  auto locate = [&](int n, int* part, int* local) {
    LocateTile(a, grouped ? slot - group * units_per_group + (n & 1) * units_per_group : slot + n * stride, part,
               local);
  };
  __syncthreads();

  // Brings slabs of this block into their ring slots (slab q into q % kStages);
  // (n, s) = tile and own-slab index of slab q. A barrier takes eight arrivals.
  // Ahead of the first multiplication every warp requests rows 2 * warp and
  // 2 * warp + 1 of each of the `count` first slabs, a bulk copy per row and lane
  // (one warp issuing a slab's sixteen copies spends about a thousand cycles in
  // that instruction, which here nothing hides); later one warp requests a whole
  // slab while the others multiply.
  const uint32_t ring_base = SharedAddress(ring);
  auto request = [&](int q, int n, int s, int r, bool announce, int rows_announced) {
    const int slab = rank + s * ks;
    int bytes;
    if constexpr (kQ4) {
      bytes = min(8, blocks - slab * 8) * kQ4KBytes;
    } else {
      // The row's last slab runs to the (16-byte padded) end of the row.
      bytes = min(S::kDataBytes, a.row_bytes - slab * S::kDataBytes);
    }
    const int at = q % kStages;
    const uint32_t bar = SharedAddress(&landed[at]);
    if (announce) {
      MbarArriveExpectTx(bar, static_cast<uint32_t>(rows_announced * bytes));
    }
    __syncwarp(__activemask());
    int part, local;
    locate(n, &part, &local);
    // Rows past the end repeat the last row; their sums are never stored.
    const int row = min(local * 16 + r, a.parts[part].rows - 1);
    const uint8_t* src = a.parts[part].w +
                         (matrix * a.parts[part].rows + static_cast<size_t>(row)) * a.row_bytes +
                         static_cast<size_t>(slab) * S::kDataBytes;
    BulkCopy(ring_base + at * S::kBytes + r * S::kRowBytes, src, static_cast<uint32_t>(bytes), bar);
  };
  auto issue_first = [&](int count) {
    const int mine = lane >> 1;   // which of the slabs this lane requests from
    if (mine < count) {
      int n = 0, s = mine;
      while (s >= slabs_mine) {
        s -= slabs_mine;
        ++n;
      }
      request(mine, n, s, 2 * warp + (lane & 1), (lane & 1) == 0, 2);
    }
  };
  auto issue = [&](int q, int n, int s) {
    if (lane < 16) {
      request(q, n, s, lane, lane < kFastWarps, 2);
    }
  };
  // (tile, own-slab index) of the next slab to request; every thread keeps it.
  int req_n = 0, req_s = 0;
  auto advance = [&]() {
    if (++req_s == slabs_mine) {
      req_s = 0;
      ++req_n;
    }
  };
  // One token: a warp reads its fragments ahead of the block's barrier, so the
  // slot is free for the slab kStages on as soon as the barrier has passed.
  // More tokens hold too many registers for that to pay (the two-token step ran
  // 7 % slower with it): the barrier comes first and frees the slot of the slab
  // before, for the slab kStages - 1 on.
  constexpr bool kEarly = TOKENS == 1;
  constexpr int kAhead = kEarly || ONE ? kStages : kStages - 1;
  {
    const int first = min(kAhead, my_slabs);
    issue_first(first);
    for (int q = 0; q < first; ++q) {
      advance();
    }
  }
  if constexpr (S::kZeros) {
    // Read only after the image's barrier below.
    for (int i = threadIdx.x * 16; i < l.plane_stride; i += kFastThreads * 16) {
      *reinterpret_cast<uint4*>(zeros + i) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  float norm_ahead[8];
  LoadNormAhead(a, norm_ahead);
  GridLaunchDependents();
  // The weights above never depend on earlier kernels; the image and y do.
  GridDependencyWait();
  // Row-split ranks: the input vector may still be on its way from the peers.
  PeerWaitBlock(a.peer_wait);
  if (a.prologue == kPrologueImage) {
    const uint32_t base = SharedAddress(smem);
    for (int at = threadIdx.x * 16; at < l.bytes; at += kFastThreads * 16) {
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(base + at), "l"(a.image + at)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
  } else {
    FillImage<TOKENS>(a, l, smem, S::kExtra,
                      a.x + static_cast<size_t>(group / (a.x_group_div > 1 ? a.x_group_div : 1)) * a.x_group_stride,
                      rank, ks, 8, norm_ahead);
  }

  float out[kNB][4];
  float off[TOKENS];
  auto clear = [&]() {
#pragma unroll
    for (int nb = 0; nb < kNB; ++nb) {
      out[nb][0] = out[nb][1] = out[nb][2] = out[nb][3] = 0.f;
    }
#pragma unroll
    for (int k = 0; k < TOKENS; ++k) {
      off[k] = 0.f;
    }
  };
  cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
  // The output rows of tile n from the eight warps' row sums in exchange buffer
  // x: thread o of the callers takes (row o / TOKENS, token o % TOKENS).
  auto total_of = [&](int x, int o) {
    const float* from = exchange + x * kFastWarps * kTileFloats + o;
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kFastWarps; ++w) {
      total += from[w * kTileFloats];
    }
    return total;
  };
  auto store = [&](int n, int o, float total) {
    int part, local;
    locate(n, &part, &local);
    const int k = o % TOKENS;
    const int row = local * 16 + o / TOKENS;
    if (row < a.parts[part].rows) {
      const size_t at = static_cast<size_t>(group) * a.y_group_stride + static_cast<size_t>(k) * a.y_stride +
                        (a.epilogue == kEpilogueSwiGlu ? 0 : a.parts[part].y_offset) + row;
      if (a.peer_out.world > 0) {
        // Row-split ranks: this rank's rows go straight into every rank's copy
        // of the full vector (plain stores over NVLink for the peers).
        for (int p = 0; p < a.peer_out.world; ++p) {
          a.peer_out.y[p][at] = total;
        }
      } else {
        a.y[at] = total;
      }
    }
  };
  // Every thread of the block (of the cluster's blocks) comes here. With the
  // SwiGLU epilogue a block's tiles alternate gate, up: the gate's sum waits in
  // a register for the up tile's.
  float held_gate = 0.f;
  auto gather = [&](int n) {
    const int o = threadIdx.x;
    if (ks == 1) {
      if (o < kTileFloats) {
        const float total = total_of(n % kExchange, o);
        if (a.epilogue != kEpilogueSwiGlu) {
          store(n, o, total);
        } else if ((n & 1) == 0) {
          held_gate = total;
        } else {
          store(n, o, SiluFast(held_gate) * total);
        }
      }
      return;
    }
    float total = o < kTileFloats ? total_of(n % kExchange, o) : 0.f;
    float* slot_in_leader = cluster.map_shared_rank(peers, 0) + ((n & 1) * 8 + rank) * kTileFloats;
    if (o < kTileFloats) {
      slot_in_leader[o] = total;
    }
    cluster.sync();
    if (rank != 0 || o >= kTileFloats) {
      return;
    }
    total = 0.f;
    for (int p = 0; p < ks; ++p) {
      total += peers[((n & 1) * 8 + p) * kTileFloats + o];
    }
    store(n, o, total);
  };
  clear();
  int n = 0, s = 0;   // tile and own-slab index being multiplied
  for (int q = 0; q < my_slabs; ++q) {
    // Slab q has landed when its barrier's phase completes (bounded: the copies
    // were issued by this block; a wait that runs out gives the slab up).
    {
      const uint32_t bar = SharedAddress(&landed[q % kStages]);
      const uint32_t parity = (q / kStages) & 1u;
      if (!MbarTryWait(bar, parity)) {
        const long long start = clock64();
        while (!MbarTryWait(bar, parity) && clock64() - start < kLandLimit) {
        }
      }
    }
    const int slab = rank + s * ks;
    const int nblk = min(8, blocks - slab * 8);
    const int b = slab * 8 + warp;
    const bool mine = warp < nblk && a.variant != 1;
    const uint8_t* data = ring + (q % kStages) * S::kBytes;
    typename std::conditional<kQ4, q4k::Q4KUnit, q6k::Q6KUnit>::type unit;
    // The block's barrier: behind it a ring slot is free (every warp is done with
    // its slab: read into registers, or multiplied) and the row sums of the tile
    // before are in the exchange buffer. Warp q % 8 requests the next slab.
    auto meet = [&]() {
      __syncthreads();
      if (q + kAhead < my_slabs) {
        if (warp == (q & 7)) {
          issue(q + kAhead, req_n, req_s);
        }
        advance();
      }
      if (s == 0 && n > 0) {
        gather(n - 1);
      }
    };
    if constexpr (!kEarly) {
      meet();
    }
    if (mine) {
      if constexpr (kQ4) {
        q4k::LoadUnit(unit, data, warp, g, t);
      } else {
        q6k::LoadUnit(unit, data, warp, nblk, g, t);
      }
    }
    if constexpr (kEarly) {
      meet();
    }
    if (mine) {
      if constexpr (kQ4) {
        q4k::Accum<TOKENS> acc;
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc.out[nb][j] = out[nb][j];
          }
        }
#pragma unroll
        for (int k = 0; k < TOKENS; ++k) {
          acc.off[k] = off[k];
        }
        q4k::MultiplyUnit<TOKENS>(unit, b, g, t, lane_plane, l, col_scale, sums, acc);
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            out[nb][j] = acc.out[nb][j];
          }
        }
#pragma unroll
        for (int k = 0; k < TOKENS; ++k) {
          off[k] = acc.off[k];
        }
      } else {
        q6k::Accum<TOKENS> acc;
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc.out[nb][j] = out[nb][j];
          }
        }
        q6k::MultiplyUnit<TOKENS>(unit, b, g, t, lane_first, lane_second, l, col_scale, sums, acc);
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            out[nb][j] = acc.out[nb][j];
          }
        }
      }
    }
    if (s == slabs_mine - 1) {
      // This warp's row sums of the tile: the columns of token k are 3k .. 3k + 2
      // (one token: every column; dead ones carry a zero factor), the Q4_K
      // offsets sit in lanes t < 2 for row g and t >= 2 for row g + 8; summed
      // over the quad.
      const int x = n % kExchange;
      float* tile = exchange + (x * kFastWarps + warp) * kTileFloats;
#pragma unroll
      for (int k = 0; k < TOKENS; ++k) {
        float lo = 0.f, hi = 0.f;
#pragma unroll
        for (int nb = 0; nb < kNB; ++nb) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int col = nb * 8 + 2 * t + j;
            const bool of_k = TOKENS == 1 || (col < kNCols && col / kLimbs == k);
            lo += of_k ? out[nb][j] : 0.f;
            hi += of_k ? out[nb][2 + j] : 0.f;
          }
        }
        lo -= t < 2 ? off[k] : 0.f;
        hi -= t < 2 ? 0.f : off[k];
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
          lo += __shfl_xor_sync(0xFFFFFFFFu, lo, o);
          hi += __shfl_xor_sync(0xFFFFFFFFu, hi, o);
        }
        if (t == 0) {
          tile[g * TOKENS + k] = lo;
          tile[(g + 8) * TOKENS + k] = hi;
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
  if (a.peer_out.world > 0 && a.peer_out.slot >= 0) {
    PeerSignal(a.peer_out);   // slot < 0: copies that nobody waits on by flag (a host mirror)
  }
}

// Lets the kernel use all the shared memory a block may have (once per device).
template <int TYPE, int TOKENS, int PER_SM, bool ONE = false>
int Configure(const gufo_cuda_ctx* ctx) {
  static bool configured[16] = {};
  if (!configured[ctx->device & 15]) {
    GUFO_CUDA_TRY(cudaFuncSetAttribute(GemvMma<TYPE, TOKENS, PER_SM, ONE>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kFastMaxShared));
    configured[ctx->device & 15] = true;
  }
  return GUFO_CUDA_OK;
}

// One token needs few enough registers for three resident blocks per SM.
template <int TOKENS>
constexpr int PerSm() { return TOKENS == 1 ? 3 : 2; }

// Whether `pairs` (gate tile, up tile) pairs each get a resident block.
template <int TYPE, int TOKENS>
bool PairsFit(const gufo_cuda_ctx* ctx, int cols, int pairs) {
  const size_t smem = SharedBytes<TYPE, TOKENS>(cols);
  if (smem > static_cast<size_t>(kFastMaxShared) || Configure<TYPE, TOKENS, PerSm<TOKENS>()>(ctx) != GUFO_CUDA_OK) {
    return false;
  }
  return pairs <= ResidentBlocks(GemvMma<TYPE, TOKENS, PerSm<TOKENS>()>, ctx->device, kFastThreads, smem, 1);
}

template <int TYPE, int TOKENS, int PER_SM>
int LaunchVariant(gufo_cuda_ctx* ctx, const FastGemvArgs& args) {
  const size_t smem = SharedBytes<TYPE, TOKENS>(args.cols);
  if (smem > static_cast<size_t>(kFastMaxShared)) {
    return GUFO_CUDA_TOO_LARGE;
  }
  {
    const int rc = Configure<TYPE, TOKENS, PER_SM>(ctx);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
  }
  int row_tiles = 0;
  for (int p = 0; p < args.nparts; ++p) {
    row_tiles += (args.parts[p].rows + 15) / 16;
  }
  FastGemvArgs launch = args;
  launch.variant = ctx->gemv_variant;
  const int slabs = (args.cols / kSuperBlock + 7) / 8;
  int grid = 1;
  if (args.group_ids != nullptr) {
    if (TYPE != GUFO_CUDA_Q4_K) {
      return Fail(GUFO_CUDA_UNSUPPORTED_TYPE, "fast gemv: grouped launches run Q4_K only");
    }
    if (args.groups <= 0 || args.tokens != 1 || args.prologue == kPrologueImage) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "fast gemv: a grouped launch takes one token and a fused input");
    }
    launch.ksplit = 1;
    grid = row_tiles * args.groups;   // one block per tile
    if (args.epilogue == kEpilogueSwiGlu) {
      if (args.nparts != 2 || args.parts[0].rows != args.parts[1].rows || args.parts[0].rows % 16 != 0) {
        return Fail(GUFO_CUDA_BAD_ARGUMENT, "fast gemv: the SwiGLU epilogue takes two parts of equal whole tiles");
      }
      grid /= 2;                      // one block per (gate tile, up tile) pair
    }
  } else if (args.epilogue == kEpilogueSwiGlu) {
    // One block per (gate tile, up tile) pair: block t takes tiles t and t + grid.
    if (args.nparts != 2 || args.parts[0].rows != args.parts[1].rows || args.parts[0].rows % 16 != 0 ||
        args.peer_out.world > 0) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "fast gemv: the SwiGLU epilogue takes two parts of equal whole tiles");
    }
    launch.ksplit = 1;
    grid = row_tiles / 2;
    if (grid > ResidentBlocks(GemvMma<TYPE, TOKENS, PER_SM>, ctx->device, kFastThreads, smem, 1)) {
      return GUFO_CUDA_TOO_LARGE;   // more tile pairs than resident blocks: the caller activates by itself
    }
  } else {
    // Few rows and several slabs per tile: split the tiles' slabs over a cluster.
    PlanFastGrid(GemvMma<TYPE, TOKENS, PER_SM>, ctx->device, kFastThreads, smem, row_tiles, slabs, &launch.ksplit,
                 &grid);
    if constexpr (TOKENS <= 2) {
      // Rows of two to four slabs whose (tile, slab) pairs do not all get a block
      // above: the one-slab form is smaller and may hold them (a 2048 x 6144 Q6_K
      // product: clusters of three blocks with one slab each instead of two blocks
      // with two and one). Only then: every further kernel that alternates with
      // the others in a decode step costs instruction-cache misses at each start
      // (the same launches ran 0.4 us slower when products that gain no wider
      // split went to this form too).
      if (slabs >= 2 && slabs <= 4 && launch.ksplit < slabs) {
        const size_t smem_one = SharedBytes<TYPE, TOKENS, true>(args.cols);
        auto* one = GemvMma<TYPE, TOKENS, PER_SM, true>;
        if (Configure<TYPE, TOKENS, PER_SM, true>(ctx) == GUFO_CUDA_OK &&
            row_tiles * slabs <= ResidentBlocks(one, ctx->device, kFastThreads, smem_one, slabs)) {
          launch.ksplit = slabs;
          launch.tiles_each = 1;
          launch.tiles_more = 0;
          GUFO_CUDA_TRY(LaunchOverlapped(one, dim3(row_tiles * slabs), dim3(kFastThreads), smem_one, ctx->stream,
                                         slabs, launch));
          ctx->launches.fetch_add(1);
          return GUFO_CUDA_OK;
        }
      }
    }
  }
  {
    // Tiles per block (ksplit == 1): block b takes tiles b, b + grid, ...
    const int total = row_tiles * (args.group_ids != nullptr ? args.groups : 1);
    launch.tiles_each = total / grid;
    launch.tiles_more = total % grid;
  }
  GUFO_CUDA_TRY(LaunchOverlapped(GemvMma<TYPE, TOKENS, PER_SM>, dim3(grid), dim3(kFastThreads), smem, ctx->stream,
                                 launch.ksplit, launch));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

template <int TYPE, int TOKENS>
int Launch(gufo_cuda_ctx* ctx, const FastGemvArgs& args) {
  return LaunchVariant<TYPE, TOKENS, PerSm<TOKENS>()>(ctx, args);
}

template <int TYPE>
bool Fits(int cols, int tokens) {
  switch (tokens) {
    case 1: return SharedBytes<TYPE, 1>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 2: return SharedBytes<TYPE, 2>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 3: return SharedBytes<TYPE, 3>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 4: return SharedBytes<TYPE, 4>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 5: return SharedBytes<TYPE, 5>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 6: return SharedBytes<TYPE, 6>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 7: return SharedBytes<TYPE, 7>(cols) <= static_cast<size_t>(kFastMaxShared);
    case 8: return SharedBytes<TYPE, 8>(cols) <= static_cast<size_t>(kFastMaxShared);
    default: return false;
  }
}

template <int TYPE>
int LaunchTokens(gufo_cuda_ctx* ctx, const FastGemvArgs& args) {
  switch (args.tokens) {
    case 1: return Launch<TYPE, 1>(ctx, args);
    case 2: return Launch<TYPE, 2>(ctx, args);
    case 3: return Launch<TYPE, 3>(ctx, args);
    case 4: return Launch<TYPE, 4>(ctx, args);
    case 5: return Launch<TYPE, 5>(ctx, args);
    case 6: return Launch<TYPE, 6>(ctx, args);
    case 7: return Launch<TYPE, 7>(ctx, args);
    case 8: return Launch<TYPE, 8>(ctx, args);
    default: return Fail(GUFO_CUDA_BAD_ARGUMENT, "fast gemv: 1 to 8 tokens per launch");
  }
}

template <int TYPE>
bool PairsFitTokens(const gufo_cuda_ctx* ctx, int cols, int tokens, int pairs) {
  switch (tokens) {
    case 1: return PairsFit<TYPE, 1>(ctx, cols, pairs);
    case 2: return PairsFit<TYPE, 2>(ctx, cols, pairs);
    case 3: return PairsFit<TYPE, 3>(ctx, cols, pairs);
    case 4: return PairsFit<TYPE, 4>(ctx, cols, pairs);
    case 5: return PairsFit<TYPE, 5>(ctx, cols, pairs);
    case 6: return PairsFit<TYPE, 6>(ctx, cols, pairs);
    case 7: return PairsFit<TYPE, 7>(ctx, cols, pairs);
    case 8: return PairsFit<TYPE, 8>(ctx, cols, pairs);
    default: return false;
  }
}

}  // namespace

// Whether a launch with the SwiGLU epilogue can give each of `pairs` tile pairs
// (rows of one part / 16) a resident thread block.
bool FastSwiGluPairsFit(const gufo_cuda_ctx* ctx, int type, int cols, int tokens, int pairs) {
  return type == GUFO_CUDA_Q4_K ? PairsFitTokens<GUFO_CUDA_Q4_K>(ctx, cols, tokens, pairs)
                                : type == GUFO_CUDA_Q6_K && PairsFitTokens<GUFO_CUDA_Q6_K>(ctx, cols, tokens, pairs);
}

// Whether `tokens` rows of `cols` values fit the shared-memory image.
bool Q4KFastFits(int cols, int tokens) { return Fits<GUFO_CUDA_Q4_K>(cols, tokens); }
bool Q6KFastFits(int cols, int tokens) { return Fits<GUFO_CUDA_Q6_K>(cols, tokens); }

// Enqueues the Q4_K / Q6_K parts of one launch (a staged image or a fused input).
int LaunchGemvQ4KFast(gufo_cuda_ctx* ctx, const FastGemvArgs& args) { return LaunchTokens<GUFO_CUDA_Q4_K>(ctx, args); }
int LaunchGemvQ6KFast(gufo_cuda_ctx* ctx, const FastGemvArgs& args) { return LaunchTokens<GUFO_CUDA_Q6_K>(ctx, args); }

}  // namespace gufo
