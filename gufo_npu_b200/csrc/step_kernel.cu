// The decode step as ONE persistent kernel (cooperative launch, one thread
// block per SM): the call sequence of qwen35::Decoder::Step
// (src/models/qwen35/decoder.cpp:478-528 in the reference) walked by every
// block from a program in device memory, with a grid-wide barrier where the
// launch chain had kernel boundaries. The reference's NPU decoder makes the same
// move, one submission per layer (src/models/qwen35_2b/npu_decoder.hpp:18-25,
// npu::Chain, src/npu/gemv.hpp:299-331).
//
// Why. A decode step of a 2B-class model is ~130 dependent operations of 2 to
// 15 MB each (plus one of 417 MB); as separate launches every one of them pays
// its own ramp and tail, and the step ran at a fifth of the HBM roofline. Weights
// (and the DeltaNet state of a layer not yet reached) never depend on the
// activations, so here a producer warp streams them into a shared-memory ring
// ahead of the consumers, across operation boundaries: while a block waits at a
// barrier, the next product's first slabs are already landing.
//
// Block layout (576 threads):
//   warps 0-7, 8-15  two teams of consumers. A team takes an operation's items
//                    (16-row tiles of a product, a DeltaNet column tile, an
//                    attention head or slice) round-robin over all teams of the
//                    grid; warp w of a team multiplies block w of each slab on
//                    the int8 tensor-core path (q4k_unit.cuh, q6k_unit.cuh).
//   warp 16          reducer: sums the eight warps' partial rows of an item in
//                    a fixed order and writes y, so consumers never meet.
//   warp 17          producer: one bulk copy (cp.async.bulk, completion on an
//                    mbarrier) per row of a slab, three slots per team.
// Every wait (mbarrier, grid barrier) is bounded by a cycle count; a wait that
// runs out leaves a code in the error word, raises the block's abort flag, and
// the block runs the rest of its control flow without waiting or working, so
// that no hardware barrier is left short of a participant.
#include "q4k_unit.cuh"
#include "q6k_unit.cuh"
#include "step_kernel.cuh"

namespace gufo {
namespace {

constexpr int kBarAll = 1;          // consumers + reducer
constexpr int kBarConsumers = 2;
constexpr int kBarTeam = 3;         // + team
constexpr int kAllThreads = (kStepConsumerWarps + 1) * 32;
constexpr int kConsumerThreads = kStepConsumerWarps * 32;
constexpr int kDeltaMaxDim = 128;
constexpr int kDeltaTileCols = 32;
constexpr int kNumBars = kStepTeams * (2 * kStepSlots + 2 * kStepExchange);

__device__ __forceinline__ void NamedSync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

struct TeamSync {
  int id;
  __device__ __forceinline__ void operator()() const { NamedSync(id, kTeamThreads); }
};

__device__ __forceinline__ void MbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ unsigned LoadAcquireGpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long GlobalTimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// The block's shared memory, carved from the dynamic allocation.
struct StepShared {
  uint8_t* region;      // staged input of a product, or the teams' scratch
  float* exchange;      // [team][kStepExchange][warp][16 rows][tokens]
  uint8_t* ring;        // [team][kStepSlots][kStepSlotBytes]
  uint32_t bars;        // shared address of the mbarriers
  volatile int* abort;
  const StepProgram* program;

  __device__ __forceinline__ uint32_t full(int team, int slot) const { return bars + 8 * (team * kStepSlots + slot); }
  __device__ __forceinline__ uint32_t empty(int team, int slot) const {
    return bars + 8 * (kStepTeams * kStepSlots + team * kStepSlots + slot);
  }
  __device__ __forceinline__ uint32_t xfull(int team, int e) const {
    return bars + 8 * (2 * kStepTeams * kStepSlots + team * kStepExchange + e);
  }
  __device__ __forceinline__ uint32_t xempty(int team, int e) const {
    return bars + 8 * (2 * kStepTeams * kStepSlots + kStepTeams * kStepExchange + team * kStepExchange + e);
  }
  __device__ __forceinline__ uint8_t* slot(int team, int s) const {
    return ring + static_cast<size_t>(team * kStepSlots + s) * kStepSlotBytes;
  }
  __device__ __forceinline__ float* xbuf(int team, int e, int tokens) const {
    return exchange + static_cast<size_t>(team * kStepExchange + e) * kTeamWarps * 16 * tokens;
  }

  // Waits for `parity` of an mbarrier for at most the program's limit, and only
  // while the block has not given up. False: the phase was not seen complete.
  __device__ __forceinline__ bool Wait(uint32_t bar, uint32_t parity, unsigned code) const {
    if (MbarTryWait(bar, parity)) {
      return true;
    }
    if (*abort != 0) {
      return false;
    }
    const long long start = clock64();
    for (;;) {
      if (MbarTryWait(bar, parity)) {
        return true;
      }
      if (*abort != 0) {
        return false;
      }
      if (clock64() - start > program->wait_limit) {
        *abort = 1;
        atomicCAS(program->sync + 2, 0u, code);
        return false;
      }
    }
  }
};


// First item of team `gg` (of `ng` teams in the grid); its items follow ng apart.
__device__ __forceinline__ int FirstItem(const StepOp& op, int gg, int ng) {
  int i = gg - op.rot;
  return i < 0 ? i + ng : i;
}

__device__ __forceinline__ void LocatePart(const StepGemv& a, int tile, int* part, int* local) {
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

__device__ __forceinline__ float Sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float Silu(float x) { return x * Sigmoid(x); }
__device__ __forceinline__ float Softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

__device__ __forceinline__ void Load8Cg(const float* p, float (&v)[8]) {
  const float4 v0 = __ldcg(reinterpret_cast<const float4*>(p));
  const float4 v1 = __ldcg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = v0.x, v[1] = v0.y, v[2] = v0.z, v[3] = v0.w;
  v[4] = v1.x, v[5] = v1.y, v[6] = v1.z, v[7] = v1.w;
}
__device__ __forceinline__ void Load8(const float* p, float (&v)[8]) {
  const float4 v0 = __ldg(reinterpret_cast<const float4*>(p));
  const float4 v1 = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = v0.x, v[1] = v0.y, v[2] = v0.z, v[3] = v0.w;
  v[4] = v1.x, v[5] = v1.y, v[6] = v1.z, v[7] = v1.w;
}
__device__ __forceinline__ void Store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// ---- the staged input of a product ------------------------------------------

// Builds the fixed-point image of a product's input (mma_common.cuh) in the
// region from the product's fused input, by the sixteen consumer warps: warp w
// converts the 256-value blocks w, w + 16, ... Activations written earlier in
// this launch by other blocks are read through L2. Block 0 (`first`) also
// writes the new residual stream, the normed rows and the position counter.
// Ends with a barrier of the consumers.
template <int TOKENS>
__device__ __noinline__ void BuildImage(const StepGemv& a, const ImageLayout& l, uint8_t* image, float extra, float* red,
                           bool first) {
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int n = a.cols;
  const int blocks = n / kSuperBlock;
  float* scale = reinterpret_cast<float*>(image + l.scale_at);
  for (int i = tid; i < blocks * l.kcols; i += kConsumerThreads) {
    if (i % l.kcols >= kLimbs * TOKENS) {
      scale[i] = 0.f;   // columns without a token keep a zero factor
    }
  }
  if (a.type == GUFO_CUDA_Q6_K) {
    // The plane of zeros of the Q6_K units (q6k_unit.cuh), behind the image.
    uint8_t* zeros = image + l.bytes;
    for (int i = tid * 16; i < l.plane_stride; i += kConsumerThreads * 16) {
      *reinterpret_cast<uint4*>(zeros + i) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  if (a.prologue == kPrologueResNorm) {
    // vec::RmsNorm (src/core/vec.hpp:57-63) of the residual stream after its
    // pending add (decoder.cpp:493,504-508); the add may come as several partial
    // vectors (a product split over K), summed here in a fixed order.
#pragma unroll 1
    for (int tok = 0; tok < TOKENS; ++tok) {
      const size_t row = static_cast<size_t>(tok) * n;
      auto residual = [&](int at, float (&v)[8]) {
        Load8Cg(a.h_in + row + at, v);
        if (a.delta != nullptr) {
          float d[8];
          Load8Cg(a.delta + row + at, d);
          for (int p = 1; p < a.delta_parts; ++p) {
            float more[8];
            Load8Cg(a.delta + static_cast<size_t>(p) * a.delta_stride + row + at, more);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              d[i] += more[i];
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[i] += d[i];
          }
        }
      };
      if (tok > 0) {
        NamedSync(kBarConsumers, kConsumerThreads);   // the sums of the token before have been read
      }
      float keep[8] = {};
      float sq = 0.f;
      for (int b = warp; b < blocks; b += kStepConsumerWarps) {
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
        red[warp] = sq;
      }
      NamedSync(kBarConsumers, kConsumerThreads);
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kStepConsumerWarps; ++w) {
        total += red[w];
      }
      const float inv = 1.0f / sqrtf(total / static_cast<float>(n) + a.eps);
      for (int b = warp; b < blocks; b += kStepConsumerWarps) {
        const int at = b * kSuperBlock + lane * 8;
        float v[8], w[8], out[8];
        if (b == warp) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[i] = keep[i];
          }
        } else {
          residual(at, v);
        }
        Load8(a.norm_w + at, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          out[i] = v[i] * inv * w[i];
        }
        if (first) {
          Store8(a.h_out + row + at, v);
          if (a.normed_out != nullptr) {
            Store8(a.normed_out + row + at, out);
          }
        }
        StageBlock(out, lane, tok, b, l, image, extra);
      }
    }
    if (first && tid == 0 && a.advance != nullptr) {
      *a.advance += TOKENS;
    }
  } else if (a.prologue == kPrologueGatedNorm) {
    // Per DeltaNet head: RMS(y) * w * silu(z) (decoder.cpp:258-263); a lane's
    // eight values lie inside one head, a head spans head_dim / 8 adjacent lanes.
    const int dk = a.gate_head_dim;
#pragma unroll 1
    for (int tok = 0; tok < TOKENS; ++tok) {
      for (int b = warp; b < blocks; b += kStepConsumerWarps) {
        const int at = b * kSuperBlock + lane * 8;
        float y[8], z[8], w[8], out[8];
        Load8Cg(a.x + static_cast<size_t>(tok) * n + at, y);
        Load8Cg(a.z + static_cast<size_t>(tok) * a.z_stride + at, z);
        Load8(a.gate_w + at % dk, w);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          ss += y[i] * y[i];
        }
        for (int o = 1; o < dk / 8; o <<= 1) {
          ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        }
        const float inv = 1.0f / sqrtf(ss / static_cast<float>(dk) + a.eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          out[i] = y[i] * inv * w[i] * Silu(z[i]);
        }
        StageBlock(out, lane, tok, b, l, image, extra);
      }
    }
  } else {
    const size_t stride = a.prologue == kPrologueSwiGlu ? 2 * static_cast<size_t>(n) : static_cast<size_t>(n);
#pragma unroll 1
    for (int tok = 0; tok < TOKENS; ++tok) {
      const float* xt = a.x + tok * stride;
      for (int b = warp; b < blocks; b += kStepConsumerWarps) {
        const int at = b * kSuperBlock + lane * 8;
        float v[8];
        Load8Cg(xt + at, v);
        if (a.prologue == kPrologueSwiGlu) {
          float up[8];
          Load8Cg(xt + n + at, up);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[i] = SiluFast(v[i]) * up[i];
          }
        }
        StageBlock(v, lane, tok, b, l, image, extra);
      }
    }
  }
  NamedSync(kBarConsumers, kConsumerThreads);
}

// ---- products -----------------------------------------------------------------

// A team's items of one product: per item the slabs' units are multiplied from
// the ring as they land, then the eight warps' row sums go to the reducer.
// `n` counts the team's ring units, `e` its items handed over, across the step.
template <int TYPE, int TOKENS>
__device__ __noinline__ void TeamGemv(const StepShared& sh, const StepOp& op, const StepGemv& a, int team, int gg, int ng,
                         unsigned& n, unsigned& e) {
  constexpr bool kQ4 = TYPE == GUFO_CUDA_Q4_K;
  constexpr int kNCols = TOKENS * kLimbs;
  constexpr int kNB = (kNCols + 7) / 8;
  const int tid = threadIdx.x - team * kTeamThreads;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const ImageLayout l = MakeImageLayout(TOKENS, a.cols, kQ4 ? 32 : 16);
  const uint8_t* image = sh.region;
  const float* col_scale = reinterpret_cast<const float*>(image + l.scale_at);
  const float* sums = reinterpret_cast<const float*>(image + l.sums_at);
  const int blocks = a.cols / kSuperBlock;
  const int spt = a.slabs_per_tile;
  // Lane planes of the two unit kinds (see the GEMV kernels).
  const uint8_t* lane_plane = image + (g % kNCols) * l.plane_stride + 8 * t;
  const uint8_t* zeros = image + l.bytes;
  const uint8_t* none = zeros + 8 * t;
  const bool one_live = (g & 3) < kNCols && ((g < 4) == (t < 2));
  const uint8_t* lane_first = TOKENS == 1 ? (one_live ? image + (g & 3) * l.plane_stride + 8 * t : none)
                                          : (t < 2 ? lane_plane : none);
  const uint8_t* lane_second = t < 2 ? none : lane_plane;

  for (int item = FirstItem(op, gg, ng); item < op.items; item += ng) {
    const int first_slab = a.split ? item % spt : 0;
    const int slabs = a.split ? 1 : spt;
    float out[kNB][4];
    float off[TOKENS];
#pragma unroll
    for (int nb = 0; nb < kNB; ++nb) {
      out[nb][0] = out[nb][1] = out[nb][2] = out[nb][3] = 0.f;
    }
#pragma unroll
    for (int k = 0; k < TOKENS; ++k) {
      off[k] = 0.f;
    }
    for (int s = first_slab; s < first_slab + slabs; ++s) {
      const int slot = n % kStepSlots;
      const bool landed = sh.Wait(sh.full(team, slot), (n / kStepSlots) & 1u, kStepErrSlotFull);
      const uint8_t* slab = sh.slot(team, slot);
      const int nblk = min(8, blocks - s * 8);
      const int b = s * 8 + warp;
      if constexpr (kQ4) {
        q4k::Q4KUnit unit;
        if (warp < nblk) {
          q4k::LoadUnit(unit, slab, warp, g, t);
        }
        __syncwarp();
        if (lane == 0) {
          MbarArrive(sh.empty(team, slot));
        }
        if (warp < nblk && landed) {
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
        }
      } else {
        q6k::Q6KUnit unit;
        if (warp < nblk) {
          q6k::LoadUnit(unit, slab, warp, nblk, g, t);
        }
        __syncwarp();
        if (lane == 0) {
          MbarArrive(sh.empty(team, slot));
        }
        if (warp < nblk && landed) {
          q6k::Accum<TOKENS> acc;
#pragma unroll
          for (int nb = 0; nb < kNB; ++nb) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              acc.out[nb][j] = out[nb][j];
            }
          }
#pragma unroll
          for (int k = 0; k < TOKENS; ++k) {
            acc.off[k] = 0.f;
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
      ++n;
    }
    // Row sums of this warp: columns of token k are 3k .. 3k + 2 (one token:
    // every live column; dead ones carry a zero factor); the Q4_K offsets sit
    // in lanes t < 2 for row g and t >= 2 for row g + 8. Summed over the quad.
    float lo[TOKENS], hi[TOKENS];
#pragma unroll
    for (int k = 0; k < TOKENS; ++k) {
      lo[k] = 0.f;
      hi[k] = 0.f;
#pragma unroll
      for (int nb = 0; nb < kNB; ++nb) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int col = nb * 8 + 2 * t + j;
          const bool mine = TOKENS == 1 || (col < kNCols && col / kLimbs == k);
          lo[k] += mine ? out[nb][j] : 0.f;
          hi[k] += mine ? out[nb][2 + j] : 0.f;
        }
      }
      lo[k] -= t < 2 ? off[k] : 0.f;
      hi[k] -= t < 2 ? 0.f : off[k];
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        lo[k] += __shfl_xor_sync(0xFFFFFFFFu, lo[k], o);
        hi[k] += __shfl_xor_sync(0xFFFFFFFFu, hi[k], o);
      }
    }
    const int x = e % kStepExchange;
    sh.Wait(sh.xempty(team, x), ((e / kStepExchange) & 1u) ^ 1u, kStepErrExchange);
    if (t == 0) {
      float* mine = sh.xbuf(team, x, TOKENS) + warp * 16 * TOKENS;
#pragma unroll
      for (int k = 0; k < TOKENS; ++k) {
        mine[g * TOKENS + k] = lo[k];
        mine[(g + 8) * TOKENS + k] = hi[k];
      }
    }
    __syncwarp();
    if (lane == 0) {
      MbarArrive(sh.xfull(team, x));
    }
    ++e;
  }
}

// The reducer warp's share of a product: for every item of the block's two
// teams, in the order each team hands them over, the sum of the eight warps'
// rows (fixed order) goes to y.
template <int TOKENS>
__device__ __noinline__ void ReduceGemv(const StepShared& sh, const StepOp& op, const StepGemv& a, int gg0, int ng,
                           unsigned (&e)[kStepTeams]) {
  const int lane = threadIdx.x & 31;
  int item[kStepTeams];
#pragma unroll
  for (int team = 0; team < kStepTeams; ++team) {
    item[team] = FirstItem(op, gg0 + team, ng);
  }
  const int spt = a.slabs_per_tile;
  long long idle_since = 0;
  bool idle = false;
  while (item[0] < op.items || item[1] < op.items) {
    bool any = false;
#pragma unroll
    for (int team = 0; team < kStepTeams; ++team) {
      if (item[team] >= op.items) {
        continue;
      }
      const int x = e[team] % kStepExchange;
      const bool ready =
          __shfl_sync(0xFFFFFFFFu, MbarTryWait(sh.xfull(team, x), (e[team] / kStepExchange) & 1u) ? 1 : 0, 0) != 0;
      if (!ready) {
        continue;
      }
      any = true;
      const int tile = a.split ? item[team] / spt : item[team];
      const int slab = a.split ? item[team] % spt : 0;
      int part, local;
      LocatePart(a, tile, &part, &local);
      if (lane < 16 * TOKENS) {
        const int k = lane % TOKENS;
        const int r = lane / TOKENS;
        const float* from = sh.xbuf(team, x, TOKENS) + r * TOKENS + k;
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kTeamWarps; ++w) {
          total += from[w * 16 * TOKENS];
        }
        const int row = local * 16 + r;
        if (row < a.parts[part].rows) {
          a.y[static_cast<size_t>(slab) * a.y_split_stride + static_cast<size_t>(k) * a.y_stride +
              a.parts[part].y_offset + row] = total;
        }
      }
      __syncwarp();
      if (lane == 0) {
        MbarArrive(sh.xempty(team, x));
      }
      ++e[team];
      item[team] += ng;
    }
    if (any) {
      idle = false;
      continue;
    }
    if (*sh.abort != 0) {
      break;
    }
    if (!idle) {
      idle = true;
      idle_since = clock64();
    } else if (clock64() - idle_since > sh.program->wait_limit) {
      *sh.abort = 1;
      atomicCAS(sh.program->sync + 2, 0u, kStepErrReducer);
      break;
    }
  }
  // Items skipped after a failure still count, so that the exchange buffers'
  // parities stay those of the consumers.
#pragma unroll
  for (int team = 0; team < kStepTeams; ++team) {
    for (; item[team] < op.items; item[team] += ng) {
      ++e[team];
    }
  }
}

// ---- Gated DeltaNet -------------------------------------------------------------

struct DeltaScratch {
  float q[kDeltaMaxDim];
  float k[kDeltaMaxDim];
  float v[kDeltaTileCols];
  float part[2][kTeamWarps][kDeltaTileCols];
  float red[3][kTeamWarps];
};

// Causal depthwise conv + SiLU of channel `ch` (decoder.cpp:178-199); the
// owner also advances the channel's window into the other buffer.
__device__ __forceinline__ float ConvChannel(const StepDelta& d, const float* conv_in, float* conv_out,
                                             int channels, int ch, bool owner) {
  const int window = d.conv_kernel - 1;
  const float* kw = d.conv_w + static_cast<size_t>(ch) * d.conv_kernel;
  const float cur = __ldcg(d.in + ch);
  float acc = __ldg(kw + window) * cur;
  for (int tap = 0; tap < window; ++tap) {
    const float old = conv_in[static_cast<size_t>(tap) * channels + ch];
    acc = fmaf(__ldg(kw + tap), old, acc);
    if (owner && tap > 0) {
      conv_out[static_cast<size_t>(tap - 1) * channels + ch] = old;
    }
  }
  if (owner) {
    conv_out[static_cast<size_t>(window - 1) * channels + ch] = cur;
  }
  return Silu(acc);
}

// A team's items of one DeltaNet layer. An item is (value head, tile of 32
// state columns): conv + SiLU + L2 norms of the head's q and k, the two gates
// from the layer's alpha / beta rows, then the delta rule (decoder.cpp:234-257)
// on the column tile the producer brought into the ring: S read once from
// shared memory into registers, S' written once to HBM. Columns evolve
// independently (src/models/qwen35/prefill_mixer.cpp:662-667). The head's
// outputs leave before the gated norm, which the output projection applies
// while it stages its input.
__device__ __noinline__ void TeamDelta(const StepShared& sh, const StepOp& op, const StepDelta& d, int team, int gg, int ng,
                          unsigned& n) {
  const int tid = threadIdx.x - team * kTeamThreads;
  const int warp = tid >> 5, lane = tid & 31;
  DeltaScratch& sc = *reinterpret_cast<DeltaScratch*>(sh.region + team * ((sizeof(DeltaScratch) + 15) / 16 * 16));
  const TeamSync sync{kBarTeam + team};
  const int dk = d.head_dim, hk = d.key_heads, hv = d.value_heads;
  const int key_dim = hk * dk;
  const int channels = 2 * key_dim + hv * dk;
  const int tiles_per_head = dk / kDeltaTileCols;
  const int rows = dk / kTeamWarps;   // state rows per lane: i = warp + 8 r
  const float* conv_in = d.conv[sh.program->parity];
  float* conv_out = d.conv[sh.program->parity ^ 1];
  for (int item = FirstItem(op, gg, ng); item < op.items; item += ng) {
    const int head = item / tiles_per_head;
    const int col0 = (item - head * tiles_per_head) * kDeltaTileCols;
    const int kh = head % hk;
    // The window of the key head's q and k channels is advanced by the first
    // value head that reads the key head, in its first tile; every tile
    // advances its own v channels.
    const bool qk_owner = head < hk && col0 == 0;
    float val = 0.f;
    if (tid < dk) {
      val = ConvChannel(d, conv_in, conv_out, channels, kh * dk + tid, qk_owner);
    } else if (tid >= kDeltaMaxDim && tid < kDeltaMaxDim + dk) {
      val = ConvChannel(d, conv_in, conv_out, channels, key_dim + kh * dk + (tid - kDeltaMaxDim), qk_owner);
    }
    float vval = 0.f;
    if (tid < kDeltaTileCols) {
      vval = ConvChannel(d, conv_in, conv_out, channels, 2 * key_dim + head * dk + col0 + tid, true);
    }
    // The head's alpha and beta rows against the layer's normed input
    // (GgufProjections serves these F32 rows, gguf_projections.cpp:162-170).
    float pa = 0.f, pb = 0.f;
    {
      const float4* xa = reinterpret_cast<const float4*>(d.gate_x);
      const float4* wa = reinterpret_cast<const float4*>(d.alpha_w + static_cast<size_t>(head) * d.cols);
      const float4* wb = reinterpret_cast<const float4*>(d.beta_w + static_cast<size_t>(head) * d.cols);
      for (int i = tid; i < d.cols / 4; i += kTeamThreads) {
        const float4 xv = __ldcg(xa + i);
        const float4 av = __ldg(wa + i), bv = __ldg(wb + i);
        pa += av.x * xv.x + av.y * xv.y + av.z * xv.z + av.w * xv.w;
        pb += bv.x * xv.x + bv.y * xv.y + bv.z * xv.z + bv.w * xv.w;
      }
    }
    const float sq = WarpSum(val * val);
    pa = WarpSum(pa);
    pb = WarpSum(pb);
    if (lane == 0) {
      sc.red[0][warp] = sq;
      sc.red[1][warp] = pa;
      sc.red[2][warp] = pb;
    }
    sync();
    float qq = 0.f, kk = 0.f, alpha = 0.f, beta = 0.f;
#pragma unroll
    for (int w = 0; w < kTeamWarps; ++w) {
      if (w < kTeamWarps / 2) {
        qq += sc.red[0][w];
      } else {
        kk += sc.red[0][w];
      }
      alpha += sc.red[1][w];
      beta += sc.red[2][w];
    }
    // L2 norms (+1e-6 under the root); q also takes 1/sqrt(dk) (decoder.cpp:200-214).
    if (tid < dk) {
      sc.q[tid] = val * ((1.0f / sqrtf(qq + 1e-6f)) * (1.0f / sqrtf(static_cast<float>(dk))));
    } else if (tid >= kDeltaMaxDim && tid < kDeltaMaxDim + dk) {
      sc.k[tid - kDeltaMaxDim] = val * (1.0f / sqrtf(kk + 1e-6f));
    }
    if (tid < kDeltaTileCols) {
      sc.v[tid] = vval;
    }
    const float decay = expf(__ldg(d.ssm_a + head) * Softplus(alpha + __ldg(d.dt_bias + head)));
    beta = Sigmoid(beta);
    sync();

    const int slot = n % kStepSlots;
    const bool landed = sh.Wait(sh.full(team, slot), (n / kStepSlots) & 1u, kStepErrSlotFull);
    const float* tile = reinterpret_cast<const float*>(sh.slot(team, slot));
    float s[kDeltaMaxDim / kTeamWarps];
#pragma unroll
    for (int r = 0; r < kDeltaMaxDim / kTeamWarps; ++r) {
      s[r] = r < rows ? tile[(warp + kTeamWarps * r) * kDeltaTileCols + lane] : 0.f;
    }
    __syncwarp();
    if (lane == 0) {
      MbarArrive(sh.empty(team, slot));
    }
    ++n;
    // Pass 1: u_j = sum_i S_ij (k_i decay).
    float u = 0.f;
#pragma unroll
    for (int r = 0; r < kDeltaMaxDim / kTeamWarps; ++r) {
      if (r < rows) {
        u = fmaf(s[r], sc.k[warp + kTeamWarps * r] * decay, u);
      }
    }
    sc.part[0][warp][lane] = u;
    sync();
    u = 0.f;
#pragma unroll
    for (int w = 0; w < kTeamWarps; ++w) {
      u += sc.part[0][w][lane];
    }
    const float delta = beta * (sc.v[lane] - u);
    // Pass 2: S'_ij = S_ij decay + k_i delta_j; y_j = sum_i S'_ij q_i.
    float* dst = d.state + (static_cast<size_t>(head) * dk) * dk + col0 + lane;
    float y = 0.f;
#pragma unroll
    for (int r = 0; r < kDeltaMaxDim / kTeamWarps; ++r) {
      if (r < rows) {
        const int i = warp + kTeamWarps * r;
        const float next = fmaf(s[r], decay, sc.k[i] * delta);
        if (landed) {
          dst[static_cast<size_t>(i) * dk] = next;
        }
        y = fmaf(next, sc.q[i], y);
      }
    }
    sc.part[1][warp][lane] = y;
    sync();
    if (warp == 0) {
      y = 0.f;
#pragma unroll
      for (int w = 0; w < kTeamWarps; ++w) {
        y += sc.part[1][w][lane];
      }
      d.y[head * dk + col0 + lane] = y;
    }
    sync();   // the scratch is reused by the team's next item
  }
}

// A team's items of one attention operation (bodies in decode_device.cuh).
__device__ __noinline__ void TeamAttention(const StepShared& sh, const StepOp& op, const AttnArgs& a, int team,
                                           int gg, int ng) {
  const int tid = threadIdx.x - team * kTeamThreads;
  AttnScratch& scratch = *reinterpret_cast<AttnScratch*>(sh.region + team * ((sizeof(AttnScratch) + 15) / 16 * 16));
  const TeamSync sync{kBarTeam + team};
  for (int item = FirstItem(op, gg, ng); item < op.items; item += ng) {
    if (op.kind == kStepAttnPrep) {
      AttnPrepBody(a, item, scratch, tid, sync);
    } else if (op.kind == kStepAttnSlice) {
      AttnSliceBody(a, item % kAttnSplits, item / kAttnSplits, scratch, tid, sync);
    } else {
      AttnMergeBody(a, item, tid);
    }
  }
}

// ---- the producer -----------------------------------------------------------------

struct Cursor {
  int op;
  int item;     // -1: the operation has not been entered yet
  int slab;
  unsigned n;   // units issued
};

// Moves the cursor of team `gg` to its next unit that has bytes to bring in
// (a slab of a product, a DeltaNet state tile). False at the end of the program.
__device__ __forceinline__ bool NextUnit(const StepProgram& p, Cursor& c, int gg, int ng, StepOp* op) {
  while (c.op < p.nops) {
    *op = p.ops[c.op];
    if (op->kind == kStepGemv || op->kind == kStepDelta) {
      if (c.item < 0) {
        c.item = FirstItem(*op, gg, ng);
        c.slab = 0;
      }
      if (c.item < op->items) {
        return true;
      }
    }
    ++c.op;
    c.item = -1;
  }
  return false;
}

__device__ __noinline__ void Producer(const StepShared& sh, int gg0, int ng) {
  const StepProgram& p = *sh.program;
  const int lane = threadIdx.x & 31;
  Cursor cur[kStepTeams];
  bool more[kStepTeams];
#pragma unroll
  for (int team = 0; team < kStepTeams; ++team) {
    cur[team] = Cursor{0, -1, 0, 0u};
    more[team] = true;
  }
  long long idle_since = 0;
  bool idle = false;
  while (more[0] || more[1]) {
    bool any = false;
#pragma unroll
    for (int team = 0; team < kStepTeams; ++team) {
      if (!more[team]) {
        continue;
      }
      Cursor& c = cur[team];
      StepOp op;
      if (!NextUnit(p, c, gg0 + team, ng, &op)) {
        more[team] = false;
        continue;
      }
      const int slot = c.n % kStepSlots;
      const bool free_slot =
          __shfl_sync(0xFFFFFFFFu, MbarTryWait(sh.empty(team, slot), ((c.n / kStepSlots) & 1u) ^ 1u) ? 1 : 0, 0) != 0;
      if (!free_slot) {
        continue;
      }
      any = true;
      const uint32_t bar = sh.full(team, slot);
      const uint32_t dst = SharedAddress(sh.slot(team, slot));
      if (op.kind == kStepGemv) {
        const StepGemv& a = p.gemv[op.arg];
        const int spt = a.slabs_per_tile;
        const int tile = a.split ? c.item / spt : c.item;
        const int slab = a.split ? c.item % spt : c.slab;
        int part, local;
        LocatePart(a, tile, &part, &local);
        int bytes, stride, offset;
        if (a.type == GUFO_CUDA_Q4_K) {
          const int nblk = min(8, a.cols / kSuperBlock - slab * 8);
          bytes = nblk * kQ4KBytes;
          stride = q4k::kSlabRowBytes;
          offset = slab * (8 * kQ4KBytes);
        } else {
          bytes = min(q6k::kSlabDataBytes, a.row_bytes - slab * q6k::kSlabDataBytes);
          stride = q6k::kSlabRowBytes;
          offset = slab * q6k::kSlabDataBytes;
        }
        if (lane == 0) {
          MbarArriveExpectTx(bar, 16u * static_cast<uint32_t>(bytes));
        }
        __syncwarp();
        if (lane < 16) {
          // Rows past the end repeat the last row; their sums are never stored.
          const int row = min(local * 16 + lane, a.parts[part].rows - 1);
          BulkCopy(dst + lane * stride, a.parts[part].w + static_cast<size_t>(row) * a.row_bytes + offset,
                   static_cast<uint32_t>(bytes), bar);
        }
        if (a.split || ++c.slab == spt) {
          c.slab = 0;
          c.item += ng;
        }
      } else {
        const StepDelta& d = p.delta[op.arg];
        const int dk = d.head_dim;
        const int tiles_per_head = dk / kDeltaTileCols;
        const int head = c.item / tiles_per_head;
        const int col0 = (c.item - head * tiles_per_head) * kDeltaTileCols;
        if (lane == 0) {
          MbarArriveExpectTx(bar, static_cast<uint32_t>(dk) * kDeltaTileCols * 4u);
        }
        __syncwarp();
        const float* src = d.state + (static_cast<size_t>(head) * dk) * dk + col0;
        for (int i = lane; i < dk; i += 32) {
          BulkCopy(dst + i * kDeltaTileCols * 4, src + static_cast<size_t>(i) * dk, kDeltaTileCols * 4u, bar);
        }
        c.item += ng;
      }
      ++c.n;
    }
    if (any) {
      idle = false;
      continue;
    }
    if (*sh.abort != 0) {
      break;
    }
    if (!idle) {
      idle = true;
      idle_since = clock64();
    } else if (clock64() - idle_since > p.wait_limit) {
      *sh.abort = 1;
      atomicCAS(p.sync + 2, 0u, kStepErrSlotEmpty);
      break;
    }
  }
  // Copies still in flight must have landed before the block may leave (after a
  // failure the consumers no longer wait for them): the last units' barriers,
  // each wait bounded by the limit alone.
#pragma unroll
  for (int team = 0; team < kStepTeams; ++team) {
    const unsigned issued = cur[team].n;
    for (unsigned k = issued > kStepSlots ? issued - kStepSlots : 0u; k < issued; ++k) {
      const long long start = clock64();
      while (!MbarTryWait(sh.full(team, k % kStepSlots), (k / kStepSlots) & 1u)) {
        if (clock64() - start > p.wait_limit) {
          break;
        }
      }
    }
  }
}

// ---- the grid barrier ---------------------------------------------------------------

// Thread 0 of a block after operation `oi`: arrives, then waits until every
// block has (bounded). The fences around it make the block's writes visible to
// the others and theirs to this block (the block's other threads meet thread 0
// at a hardware barrier before and after).
__device__ void GridBarrier(const StepShared& sh, int oi) {
  const StepProgram& p = *sh.program;
  __threadfence();
  if (!(p.skip_arrival_at == oi && blockIdx.x == 0)) {
    atomicAdd(p.sync, 1u);
  }
  const unsigned target = static_cast<unsigned>(oi + 1) * gridDim.x;
  if (*sh.abort == 0) {
    const long long start = clock64();
    unsigned polls = 0;
    while (LoadAcquireGpu(p.sync) < target) {
      if ((++polls & 31u) == 0) {
        if (clock64() - start > p.wait_limit) {
          atomicCAS(p.sync + 2, 0u, kStepErrGridBarrier);
          *sh.abort = 1;
          break;
        }
        if (*reinterpret_cast<volatile unsigned*>(p.sync + 2) != 0) {
          *sh.abort = 1;   // another block gave up
          break;
        }
      }
    }
  }
  __threadfence();
  if (blockIdx.x == 0 && p.stamps != nullptr) {
    p.stamps[oi + 1] = GlobalTimer();
  }
}

template <int TOKENS>
__global__ void __launch_bounds__(kStepThreads, 1)
StepKernel(const __grid_constant__ StepProgram p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red[kStepConsumerWarps];
  __shared__ int abort_flag;
  // The abort flag as thread 0 saw it at the last operation boundary: every
  // consumer takes the same branch around an operation's team barriers.
  __shared__ int op_abort;
  StepShared sh;
  sh.region = smem;
  sh.exchange = reinterpret_cast<float*>(smem + p.region_bytes);
  sh.ring = reinterpret_cast<uint8_t*>(sh.exchange) + kStepTeams * kStepExchange * kTeamWarps * 16 * TOKENS * 4;
  sh.bars = SharedAddress(sh.ring + kStepTeams * kStepSlots * kStepSlotBytes);
  sh.abort = &abort_flag;
  sh.program = &p;
  const int warp = threadIdx.x >> 5;
  const int ng = static_cast<int>(gridDim.x) * kStepTeams;
  const int gg0 = static_cast<int>(blockIdx.x) * kStepTeams;
  if (threadIdx.x == 0) {
    // A failure of an earlier launch that nobody cleared: do not start.
    abort_flag = *reinterpret_cast<volatile unsigned*>(p.sync + 2) != 0 ? 1 : 0;
    op_abort = abort_flag;
    for (int team = 0; team < kStepTeams; ++team) {
      for (int s = 0; s < kStepSlots; ++s) {
        MbarInit(sh.full(team, s), 1);
        MbarInit(sh.empty(team, s), kTeamWarps);
      }
      for (int x = 0; x < kStepExchange; ++x) {
        MbarInit(sh.xfull(team, x), kTeamWarps);
        MbarInit(sh.xempty(team, x), 1);
      }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (blockIdx.x == 0 && p.stamps != nullptr) {
      p.stamps[0] = GlobalTimer();
    }
  }
  __syncthreads();

  if (warp == kStepProducerWarp) {
    Producer(sh, gg0, ng);
    return;
  }
  if (warp == kStepReducerWarp) {
    unsigned e[kStepTeams] = {0u, 0u};
    for (int oi = 0; oi < p.nops; ++oi) {
      const StepOp op = p.ops[oi];
      if (op.kind == kStepGemv) {
        ReduceGemv<TOKENS>(sh, op, p.gemv[op.arg], gg0, ng, e);
      }
      NamedSync(kBarAll, kAllThreads);
      NamedSync(kBarAll, kAllThreads);
    }
    return;
  }

  const int team = warp / kTeamWarps;
  const int gg = gg0 + team;
  const int tid = threadIdx.x - team * kTeamThreads;
  unsigned n = 0, e = 0;
  for (int oi = 0; oi < p.nops; ++oi) {
    const StepOp op = p.ops[oi];
    if (op_abort == 0) {
      switch (op.kind) {
        case kStepEmbed:
          if (FirstItem(op, gg, ng) < op.items) {
            EmbedBody(p.embed, tid);
          }
          break;
        case kStepGemv: {
          const StepGemv& a = p.gemv[op.arg];
          const bool work = FirstItem(op, gg0, ng) < op.items || FirstItem(op, gg0 + 1, ng) < op.items;
          if (work || blockIdx.x == 0) {
            const bool q4 = a.type == GUFO_CUDA_Q4_K;
            const ImageLayout l = MakeImageLayout(TOKENS, a.cols, q4 ? 32 : 16);
            BuildImage<TOKENS>(a, l, sh.region, q4 ? 1.0f / 16.0f : 0.25f, red, blockIdx.x == 0);
          }
          if (a.type == GUFO_CUDA_Q4_K) {
            TeamGemv<GUFO_CUDA_Q4_K, TOKENS>(sh, op, a, team, gg, ng, n, e);
          } else {
            TeamGemv<GUFO_CUDA_Q6_K, TOKENS>(sh, op, a, team, gg, ng, n, e);
          }
          break;
        }
        case kStepDelta:
          TeamDelta(sh, op, p.delta[op.arg], team, gg, ng, n);
          break;
        case kStepAttnPrep:
        case kStepAttnSlice:
        case kStepAttnMerge:
          TeamAttention(sh, op, p.attn[op.arg], team, gg, ng);
          break;
        default:
          break;
      }
    }
    NamedSync(kBarAll, kAllThreads);
    if (threadIdx.x == 0) {
      GridBarrier(sh, oi);
      op_abort = abort_flag;
    }
    NamedSync(kBarAll, kAllThreads);
  }
  if (threadIdx.x == 0) {
    // The last block out clears the counters for the next launch.
    if (atomicAdd(p.sync + 1, 1u) == gridDim.x - 1) {
      p.sync[0] = 0;
      p.sync[1] = 0;
    }
  }
}

}  // namespace


int StepImageBytes(int type, int cols) {
  const ImageLayout l = MakeImageLayout(kStepMaxTokens, cols, type == GUFO_CUDA_Q4_K ? 32 : 16);
  return l.bytes + (type == GUFO_CUDA_Q6_K ? (l.plane_stride + 15) / 16 * 16 : 0);
}

int StepScratchBytes() {
  const size_t attn = (sizeof(AttnScratch) + 15) / 16 * 16;
  const size_t delta = (sizeof(DeltaScratch) + 15) / 16 * 16;
  return static_cast<int>(kStepTeams * (attn > delta ? attn : delta));
}

size_t StepSharedBytes(int region_bytes) {
  return static_cast<size_t>(region_bytes) + kStepTeams * kStepExchange * kTeamWarps * 16 * kStepMaxTokens * 4 +
         static_cast<size_t>(kStepTeams) * kStepSlots * kStepSlotBytes + kNumBars * 8;
}

int StepGridBlocks(int device, int region_bytes) {
  const size_t smem = StepSharedBytes(region_bytes);
  int limit = 0, sms = 0, cooperative = 0;
  if (cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (cooperative == 0 || smem > static_cast<size_t>(limit)) {
    return 0;
  }
  if (cudaFuncSetAttribute(StepKernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
      cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, StepKernel<1>, kStepThreads, smem) != cudaSuccess ||
      per_sm < 1) {
    cudaGetLastError();
    return 0;
  }
  return sms;
}

int LaunchStep(gufo_cuda_ctx* ctx, const StepProgram& program, int grid) {
  const size_t smem = StepSharedBytes(program.region_bytes);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kStepThreads);
  config.dynamicSmemBytes = smem;
  config.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  GUFO_CUDA_TRY(cudaLaunchKernelEx(&config, StepKernel<1>, program));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

}  // namespace gufo
