// All-gather of row-split products over NVLink peer memory, for the ranks of a
// row-split decode step (one process per GPU): every rank stores its slice of a
// stage's outputs straight into every rank's copy of the full vector and raises
// a flag there; a rank is done when the flags of all the others have arrived.
// One small kernel per gather, captured in the step's graph like any other.
//
// Each rank owns an arena (one cudaMalloc allocation) opened by the others
// through CUDA IPC. The first kPeerHeaderBytes hold the flags the peers raise
// (64 bytes apart), the gather count, the count of finished blocks and an error
// word; the full vectors live behind them at the same offsets on every rank.
//
// Every wait is bounded: a flag that does not arrive within the limit sets the
// error word (gufo_cuda_peer_group_status returns GUFO_CUDA_TIMEOUT) and the
// kernel returns.
#include <cstring>

#include "peer.cuh"

namespace gufo {
namespace {

constexpr int kPeerThreads = 256;

struct PeerGatherArgs {
  uint8_t* arena[kMaxPeers];
  int rank;
  int world;
  const float* src;      // this rank's slice
  size_t offset;         // of the full vector in every arena, bytes
  unsigned slice;        // floats per rank
  long long limit;       // clock cycles a flag may take
};

// Block b serves peer b: it stores this rank's slice into b's arena, raises this
// rank's flag there, then waits for b's flag here.
__global__ void __launch_bounds__(kPeerThreads)
PeerAllGatherKernel(const __grid_constant__ PeerGatherArgs a) {
  GridLaunchDependents();
  GridDependencyWait();   // the slice was written by the kernel before this one
  const int peer = blockIdx.x;
  unsigned* header = reinterpret_cast<unsigned*>(a.arena[a.rank]);
  // The same for every block: the count moves only when the last block leaves.
  const unsigned turn = *reinterpret_cast<volatile unsigned*>(header + kCountWord) + 1;
  float* dst = reinterpret_cast<float*>(a.arena[peer] + a.offset) + static_cast<size_t>(a.rank) * a.slice;
  if (a.slice % 4 == 0) {
    const float4* src4 = reinterpret_cast<const float4*>(a.src);
    float4* dst4 = reinterpret_cast<float4*>(dst);
    for (unsigned i = threadIdx.x; i < a.slice / 4; i += kPeerThreads) {
      dst4[i] = src4[i];
    }
  } else {
    for (unsigned i = threadIdx.x; i < a.slice; i += kPeerThreads) {
      dst[i] = a.src[i];
    }
  }
  // The barrier orders the block's stores before thread 0's release at system
  // scope, which is cumulative: one fence for the block instead of one per thread
  // and another for the flag.
  __syncthreads();
  if (threadIdx.x == 0) {
    StoreReleaseSys(reinterpret_cast<unsigned*>(a.arena[peer]) + kFlagStride * a.rank, turn);
    const unsigned* mine = header + kFlagStride * peer;
    // After a first failure the later gathers of the step give up at once.
    const long long limit = *reinterpret_cast<volatile unsigned*>(header + kErrorWord) != 0 ? 0 : a.limit;
    const long long start = clock64();
    // Flags only grow; the difference copes with the counter wrapping.
    while (static_cast<int>(LoadAcquireSys(mine) - turn) < 0) {
      if (clock64() - start > limit) {
        atomicExch(header + kErrorWord, 1u);
        break;
      }
    }
    if (atomicAdd(header + kFinishedWord, 1u) == static_cast<unsigned>(a.world - 1)) {
      header[kFinishedWord] = 0;
      __threadfence();
      header[kCountWord] = turn;
    }
  }
}

// Waits for a slot's rows on behalf of kernels that do not wait themselves.
__global__ void __launch_bounds__(32)
PeerWaitKernel(const __grid_constant__ PeerWait w) {
  GridLaunchDependents();
  GridDependencyWait();
  PeerWaitBlock(w);
}

}  // namespace

PeerWait MakePeerWait(const gufo_cuda_peer_group* g, int slot) {
  PeerWait w{};
  w.header = reinterpret_cast<const unsigned*>(g->arena[g->rank]);
  w.world = g->world;
  w.slot = slot;
  w.limit = g->limit;
  return w;
}

}  // namespace gufo

using gufo::Fail;

extern "C" {

int gufo_cuda_ipc_export(gufo_cuda_ctx* ctx, const void* device_ptr, void* handle) {
  if (ctx == nullptr || device_ptr == nullptr || handle == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "ipc_export: null pointer");
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == GUFO_CUDA_IPC_HANDLE_BYTES, "handle size");
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  GUFO_CUDA_TRY(cudaIpcGetMemHandle(&h, const_cast<void*>(device_ptr)));
  std::memcpy(handle, &h, sizeof(h));
  return GUFO_CUDA_OK;
}

namespace {

// Common part of the two ways to create a group: `handles` (IPC handles of all
// ranks, another process each) or `arenas` (device pointers this process can
// already reach: its own allocations, or peers' with peer access enabled).
int CreatePeerGroup(gufo_cuda_ctx* ctx, int rank, int world, void* own_arena, size_t arena_bytes,
                    const void* handles, void* const* arenas, gufo_cuda_peer_group** out) {
  if (ctx == nullptr || own_arena == nullptr || (handles == nullptr && arenas == nullptr) || out == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_group_create: null pointer");
  }
  *out = nullptr;
  if (world < 1 || world > gufo::kMaxPeers || rank < 0 || rank >= world) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_group_create: 1 to 8 ranks, rank inside");
  }
  if (arena_bytes <= GUFO_CUDA_PEER_HEADER_BYTES || (reinterpret_cast<uintptr_t>(own_arena) & 255) != 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_group_create: the arena must exceed its header and be 256-byte aligned");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  auto* g = new gufo_cuda_peer_group();
  g->ctx = ctx;
  g->rank = rank;
  g->world = world;
  g->arena_bytes = arena_bytes;
  cudaDeviceGetAttribute(&g->khz, cudaDevAttrClockRate, ctx->device);
  if (g->khz <= 0) {
    g->khz = 1000000;
  }
  g->limit = static_cast<long long>(g->khz) * 4000;   // about four seconds of SM clocks
  for (int r = 0; r < world; ++r) {
    if (r == rank) {
      g->arena[r] = static_cast<uint8_t*>(own_arena);
      continue;
    }
    if (arenas != nullptr) {
      if (arenas[r] == nullptr || (reinterpret_cast<uintptr_t>(arenas[r]) & 255) != 0) {
        delete g;
        return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_group_create: every rank's arena must be given, 256-byte aligned");
      }
      g->arena[r] = static_cast<uint8_t*>(arenas[r]);
      continue;
    }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const uint8_t*>(handles) + static_cast<size_t>(r) * sizeof(h), sizeof(h));
    void* opened = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&opened, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      for (int q = 0; q < r; ++q) {
        if (g->opened[q]) {
          cudaIpcCloseMemHandle(g->arena[q]);
        }
      }
      delete g;
      return gufo::CudaFail(e, "cudaIpcOpenMemHandle");
    }
    g->arena[r] = static_cast<uint8_t*>(opened);
    g->opened[r] = true;
  }
  // The whole arena starts at zero on every rank, flags, counts and the error
  // word included, before this call returns: the caller lets all ranks pass a
  // barrier between creating the group and the first gather, so no peer can
  // store a slice into this arena before it has been cleared (clearing a vector
  // later, once a faster rank may already have written its slice and raised its
  // flag, would wipe the slice and keep the flag).
  GUFO_CUDA_TRY(cudaMemsetAsync(own_arena, 0, arena_bytes, ctx->stream));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  *out = g;
  return GUFO_CUDA_OK;
}

}  // namespace

int gufo_cuda_peer_group_create(gufo_cuda_ctx* ctx, int rank, int world, void* own_arena, size_t arena_bytes,
                                const void* handles, gufo_cuda_peer_group** out) {
  if (handles == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_group_create: null pointer");
  }
  return CreatePeerGroup(ctx, rank, world, own_arena, arena_bytes, handles, nullptr, out);
}

int gufo_cuda_peer_group_create_local(gufo_cuda_ctx* ctx, int rank, int world, void* const* arenas,
                                      size_t arena_bytes, gufo_cuda_peer_group** out) {
  if (arenas == nullptr || world < 1 || world > gufo::kMaxPeers || rank < 0 || rank >= world) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_group_create_local: arenas of 1 to 8 ranks, rank inside");
  }
  return CreatePeerGroup(ctx, rank, world, arenas[rank], arena_bytes, nullptr, arenas, out);
}

int gufo_cuda_peer_group_set_limit(gufo_cuda_peer_group* g, int64_t microseconds) {
  if (g == nullptr || microseconds < 1 || microseconds > 60 * 1000000ll) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_group_set_limit: a group and 1 us to 60 s");
  }
  std::lock_guard<std::mutex> lock(g->ctx->mu);
  g->limit = static_cast<long long>(g->khz) * microseconds / 1000;   // kHz * us / 1000 = cycles
  return GUFO_CUDA_OK;
}

int gufo_cuda_peer_group_reset(gufo_cuda_peer_group* g) {
  if (g == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_group_reset: null group");
  }
  gufo_cuda_ctx* ctx = g->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  GUFO_CUDA_TRY(cudaMemsetAsync(g->arena[g->rank], 0, GUFO_CUDA_PEER_HEADER_BYTES, ctx->stream));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  return GUFO_CUDA_OK;
}

int gufo_cuda_peer_group_destroy(gufo_cuda_peer_group* g) {
  if (g == nullptr) {
    return GUFO_CUDA_OK;
  }
  cudaSetDevice(g->ctx->device);
  cudaStreamSynchronize(g->ctx->stream);
  for (int r = 0; r < g->world; ++r) {
    if (g->opened[r]) {
      cudaIpcCloseMemHandle(g->arena[r]);
    }
  }
  delete g;
  return GUFO_CUDA_OK;
}

int gufo_cuda_peer_allgather_device(gufo_cuda_peer_group* g, const float* local_src, size_t arena_offset,
                                    size_t slice_floats) {
  if (g == nullptr || local_src == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_allgather: null pointer");
  }
  if (slice_floats == 0 || slice_floats > 0xFFFFFFFFu || arena_offset < GUFO_CUDA_PEER_HEADER_BYTES ||
      arena_offset % 16 != 0 || (reinterpret_cast<uintptr_t>(local_src) & 15) != 0 ||
      arena_offset + slice_floats * 4 * g->world > g->arena_bytes) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_allgather: the full vector must lie inside the arena, 16-byte aligned");
  }
  gufo_cuda_ctx* ctx = g->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  gufo::PeerGatherArgs a{};
  for (int r = 0; r < g->world; ++r) {
    a.arena[r] = g->arena[r];
  }
  a.rank = g->rank;
  a.world = g->world;
  a.src = local_src;
  a.offset = arena_offset;
  a.slice = static_cast<unsigned>(slice_floats);
  a.limit = g->limit;
  GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::PeerAllGatherKernel, dim3(g->world), dim3(gufo::kPeerThreads), 0,
                                       ctx->stream, 1, a));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

int gufo_cuda_peer_wait_device(gufo_cuda_peer_group* g, int slot) {
  if (g == nullptr || slot < 0 || slot >= gufo::kPeerSlots) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_wait: a group and a slot below 8");
  }
  gufo_cuda_ctx* ctx = g->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::PeerWaitKernel, dim3(1), dim3(32), 0, ctx->stream, 1,
                                       gufo::MakePeerWait(g, slot)));
  ctx->launches.fetch_add(1);
  return GUFO_CUDA_OK;
}

int gufo_cuda_peer_group_status(gufo_cuda_peer_group* g) {
  if (g == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "peer_group_status: null group");
  }
  gufo_cuda_ctx* ctx = g->ctx;
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  unsigned error = 0;
  GUFO_CUDA_TRY(cudaMemcpyAsync(&error, g->arena[g->rank] + gufo::kErrorWord * 4, 4, cudaMemcpyDeviceToHost,
                                ctx->stream));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  if (error != 0) {
    return Fail(GUFO_CUDA_TIMEOUT, "peer_allgather: a peer's flag did not arrive within the limit");
  }
  return GUFO_CUDA_OK;
}

}  // extern "C"
