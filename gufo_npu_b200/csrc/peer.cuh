// Layout of a peer arena's header and the device side of the flag protocol of
// the row-split ranks (peer.cu): shared by the gather kernel, the products that
// store their rows into the peers' arenas themselves (gemv_mma.cu) and the
// kernels that wait for such rows.
#pragma once

#include "common.cuh"

namespace gufo {

constexpr int kFlagStride = 16;        // words between two peers' flags (the separate gather kernel)
constexpr int kCountWord = 256;        // gathers completed by this rank
constexpr int kFinishedWord = 257;     // blocks of the running gather that are done
constexpr int kErrorWord = 258;
// Products that gather by themselves: per vector slot s, this rank's count of
// gathers sent, the turn its last product announced, its blocks that are done,
// and one flag per peer (8 words apart).
constexpr int kPeerSlots = 8;
constexpr int kSentWord = 260;         // + s
constexpr int kTurnWord = 270;         // + s
constexpr int kDoneWord = 280;         // + s
constexpr int kSlotFlags = 512;        // + 64 s + 8 peer

__device__ __forceinline__ void StoreReleaseSys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned LoadAcquireSys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Called by every thread of a block after the block's last store of a product
// with peer outputs: the last block of the grid announces the turn and raises
// this rank's flag in every arena. The release at system scope is cumulative
// over the grid's stores (each block fenced before it counted itself off).
__device__ __forceinline__ void PeerSignal(const PeerOut& out) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned* mine = out.header[out.rank];
    __threadfence();
    if (atomicAdd(mine + kDoneWord + out.slot, 1u) == gridDim.x - 1) {
      mine[kDoneWord + out.slot] = 0;
      const unsigned turn = mine[kSentWord + out.slot] + 1;
      mine[kSentWord + out.slot] = turn;
      mine[kTurnWord + out.slot] = turn;
      __threadfence_system();
      for (int p = 0; p < out.world; ++p) {
        StoreReleaseSys(out.header[p] + kSlotFlags + 64 * out.slot + 8 * out.rank, turn);
      }
    }
  }
}

// Thread 0 of the calling block waits until every rank's rows of the slot's
// current turn have arrived (bounded; a wait that runs out sets the error word
// and later waits give up at once); the block's other threads wait at the
// barrier. Call after the grid-dependency wait: the turn was announced by an
// earlier kernel of this stream.
__device__ __forceinline__ void PeerWaitBlock(const PeerWait& w) {
  if (w.header == nullptr) {
    return;
  }
  if (threadIdx.x == 0) {
    const unsigned turn = *reinterpret_cast<const volatile unsigned*>(w.header + kTurnWord + w.slot);
    const long long limit = *reinterpret_cast<const volatile unsigned*>(w.header + kErrorWord) != 0 ? 0 : w.limit;
    const long long start = clock64();
    for (int p = 0; p < w.world; ++p) {
      const unsigned* flag = w.header + kSlotFlags + 64 * w.slot + 8 * p;
      // Flags only grow; the difference copes with the counter wrapping.
      while (static_cast<int>(LoadAcquireSys(flag) - turn) < 0) {
        if (clock64() - start > limit) {
          atomicExch(const_cast<unsigned*>(w.header) + kErrorWord, 1u);
          break;
        }
      }
    }
  }
  __syncthreads();
}

}  // namespace gufo

struct gufo_cuda_peer_group {
  gufo_cuda_ctx* ctx = nullptr;
  int rank = 0;
  int world = 0;
  uint8_t* arena[gufo::kMaxPeers] = {};
  bool opened[gufo::kMaxPeers] = {};   // mapped through CUDA IPC (closed at destroy)
  size_t arena_bytes = 0;
  long long limit = 0;
  int khz = 0;
};
