// Device bodies of the small decode-step operations (embedding row, decode
// attention over the fp16 cache), written for one team of kTeamThreads threads
// and a caller-supplied barrier among that team. The stand-alone kernels of
// decoder.cu run them with one thread block per team and __syncthreads; the
// persistent decode-step kernel (step_kernel.cu) runs them with a team of eight
// warps inside a larger block and a named barrier.
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"

namespace gufo {

constexpr int kTeamThreads = 256;
constexpr int kTeamWarps = kTeamThreads / 32;
constexpr int kAttnSplits = 32;     // position slices per KV head
constexpr int kMaxGroup = 8;        // query heads per KV head
constexpr int kMaxPerLane = 8;      // head_dim / 32

// The barrier of a team that is a whole thread block.
struct BlockSync {
  __device__ __forceinline__ void operator()() const { __syncthreads(); }
};

// h = dequantized row *token of the embedding matrix (quant::Dequantize of one
// row, src/models/qwen35/decoder.cpp:486-489).
struct EmbedArgs {
  const uint8_t* data;
  int type;
  int row_bytes;
  int cols;
  const int* token;
  float* h;
};

struct AttnArgs {
  int heads, kv_heads, head_dim, rope_dim, max_positions;
  float rms_eps;
  const int* position;
  const float* in;          // [q and gate (2 heads hd, per head q | gate) | k | v]
  const float* q_norm;
  const float* k_norm;
  const float* inv_freq;    // [rope_dim / 2]
  __half* keys;             // [max_positions][kv_heads * hd]
  __half* values;
  float* queries;           // [heads][hd]
  float* partials;          // [kv_heads][splits][group][hd + 2]
  float* ctx;               // [heads][hd]
  int offset = 0;           // the token sits at *position + offset
};

// Shared memory of one team running the attention bodies.
struct AttnScratch {
  float reduce[kTeamWarps];
  float vec[kMaxPerLane * 32];
  float q[kMaxGroup][kMaxPerLane * 32];
  float merge_m[kTeamWarps];
  float merge_l[kTeamWarps];
  float merge_acc[kTeamWarps][kMaxPerLane * 32];
};

__device__ __forceinline__ float SigmoidDev(float x) { return 1.0f / (1.0f + expf(-x)); }

// Sum of one value per team thread; result to every thread. `tid` in [0, kTeamThreads).
template <typename Sync>
__device__ __forceinline__ float TeamSum(float v, float* reduce, int tid, Sync sync) {
  v = WarpSum(v);
  sync();
  if ((tid & 31) == 0) {
    reduce[tid >> 5] = v;
  }
  sync();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kTeamWarps; ++w) {
    total += reduce[w];
  }
  return total;
}

__device__ __forceinline__ void EmbedBody(const EmbedArgs& a, int tid) {
  const uint8_t* row = a.data + static_cast<size_t>(*a.token) * a.row_bytes;
  const int blocks = a.cols / kSuperBlock;
  if (a.type == GUFO_CUDA_Q4_K) {
    for (int item = tid; item < blocks * 32; item += kTeamThreads) {
      const int b = item >> 5, word = item & 31, p = word >> 3, c = word & 7;
      const uint32_t* block = reinterpret_cast<const uint32_t*>(row + b * kQ4KBytes);
      const uint32_t dd = block[0];
      const float d = HalfBitsToFloat(static_cast<uint16_t>(dd & 0xFFFF));
      const float dmin = HalfBitsToFloat(static_cast<uint16_t>(dd >> 16));
      int sc_lo, m_lo, sc_hi, m_hi;
      ScaleMinK4(2 * p, block[1], block[2], block[3], &sc_lo, &m_lo);
      ScaleMinK4(2 * p + 1, block[1], block[2], block[3], &sc_hi, &m_hi);
      const float d1 = __fmul_rn(d, static_cast<float>(sc_lo)), m1 = __fmul_rn(dmin, static_cast<float>(m_lo));
      const float d2 = __fmul_rn(d, static_cast<float>(sc_hi)), m2 = __fmul_rn(dmin, static_cast<float>(m_hi));
      const uint32_t q = block[4 + word];
      float* out = a.h + b * kSuperBlock + 64 * p + 4 * c;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[i] = __fsub_rn(__fmul_rn(d1, static_cast<float>((q >> (8 * i)) & 0xF)), m1);
        out[32 + i] = __fsub_rn(__fmul_rn(d2, static_cast<float>((q >> (8 * i + 4)) & 0xF)), m2);
      }
    }
  } else if (a.type == GUFO_CUDA_Q6_K) {
    for (int item = tid; item < blocks * 64; item += kTeamThreads) {
      const int b = item >> 6, half = (item >> 5) & 1, l = item & 31;
      const Q6KBlock block = Q6KBlockAt(row, blocks, b);
      const uint8_t* ql = block.ql + 64 * half;
      const uint8_t* qh = block.qh + 32 * half;
      const int8_t* sc = block.sc + 8 * half + (l >> 4);
      const float d = HalfBitsToFloat(*reinterpret_cast<const uint16_t*>(block.d));
      const int x = ql[l], c = ql[l + 32], h = qh[l];
      float* out = a.h + b * kSuperBlock + 128 * half + l;
      out[0] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[0])), static_cast<float>(((x & 0xF) | ((h & 3) << 4)) - 32));
      out[32] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[2])), static_cast<float>(((c & 0xF) | (((h >> 2) & 3) << 4)) - 32));
      out[64] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[4])), static_cast<float>(((x >> 4) | (((h >> 4) & 3) << 4)) - 32));
      out[96] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[6])), static_cast<float>(((c >> 4) | (((h >> 6) & 3) << 4)) - 32));
    }
  } else {
    for (int i = tid; i < a.cols; i += kTeamThreads) {
      a.h[i] = reinterpret_cast<const float*>(row)[i];
    }
  }
}

// q/k RMSNorm and RoPE; appends k and v to the cache in fp16
// (decoder.cpp:280-323). `head` < heads: query head; then one per KV head.
// Reads of the input row go through L2 (__ldcg): another block may have
// written it earlier in the same kernel.
template <typename Sync>
__device__ __forceinline__ void AttnPrepBody(const AttnArgs& a, int head, AttnScratch& s, int tid, Sync sync) {
  const int hd = a.head_dim;
  const int half = a.rope_dim / 2;
  const int pos = *a.position + a.offset;
  const bool is_query = head < a.heads;
  const int kh = head - a.heads;
  const float* x = is_query ? a.in + static_cast<size_t>(head) * 2 * hd
                            : a.in + static_cast<size_t>(a.heads) * 2 * hd + kh * hd;
  const float* w = is_query ? a.q_norm : a.k_norm;
  const int e = tid;
  const float v = e < hd ? __ldcg(x + e) : 0.f;
  const float total = TeamSum(v * v, s.reduce, tid, sync);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(hd) + a.rms_eps);
  if (e < hd) {
    s.vec[e] = v * inv * w[e];
  }
  sync();
  float out = e < hd ? s.vec[e] : 0.f;
  if (e < 2 * half) {
    const int i = e < half ? e : e - half;
    const double angle = static_cast<double>(pos) * static_cast<double>(a.inv_freq[i]);
    const float cs = static_cast<float>(cos(angle));
    const float sn = static_cast<float>(sin(angle));
    const float lo = s.vec[i], hi = s.vec[i + half];
    out = e < half ? lo * cs - hi * sn : lo * sn + hi * cs;
  }
  if (e < hd) {
    if (is_query) {
      a.queries[head * hd + e] = out;
    } else {
      const size_t at = (static_cast<size_t>(pos) * a.kv_heads + kh) * hd + e;
      a.keys[at] = __float2half_rn(out);
      const float val = __ldcg(a.in + static_cast<size_t>(a.heads) * 2 * hd + a.kv_heads * hd + kh * hd + e);
      a.values[at] = __float2half_rn(val);
    }
  }
  sync();   // the scratch may be reused by the team's next item
}

// `per` consecutive fp16 values at p (aligned to their total size when per is
// 2, 4 or 8) as floats, read through L2; out[per..] = 0.
__device__ __forceinline__ void LoadHalves(const __half* p, int per, float (&out)[kMaxPerLane]) {
  unsigned short h[kMaxPerLane] = {};
  if (per == 8) {
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(p));
    h[0] = v.x & 0xFFFF, h[1] = v.x >> 16, h[2] = v.y & 0xFFFF, h[3] = v.y >> 16;
    h[4] = v.z & 0xFFFF, h[5] = v.z >> 16, h[6] = v.w & 0xFFFF, h[7] = v.w >> 16;
  } else if (per == 4) {
    const uint2 v = __ldcg(reinterpret_cast<const uint2*>(p));
    h[0] = v.x & 0xFFFF, h[1] = v.x >> 16, h[2] = v.y & 0xFFFF, h[3] = v.y >> 16;
  } else if (per == 2) {
    const unsigned v = __ldcg(reinterpret_cast<const unsigned*>(p));
    h[0] = v & 0xFFFF, h[1] = v >> 16;
  } else {
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      if (i < per) {
        h[i] = __ldcg(reinterpret_cast<const unsigned short*>(p) + i);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    out[i] = i < per ? __half2float(__ushort_as_half(h[i])) : 0.f;
  }
}

// Where element e of a query sits in AttnScratch::q: lane e / per reads its
// elements at i * 32 + lane, one bank per lane.
__device__ __forceinline__ int QuerySlot(int e, int per) { return (e % per) * 32 + e / per; }

// One slice of the cached positions for one KV head and the query heads that
// share it: partial softmax (weighted values, max, sum) per query head (the
// split-K jobs of decoder.cpp:326-381).
template <typename Sync>
__device__ __forceinline__ void AttnSliceBody(const AttnArgs& a, int split, int kh, AttnScratch& s, int tid,
                                              Sync sync) {
  const int hd = a.head_dim;
  const int per = hd / 32;
  const int group = a.heads / a.kv_heads;
  const int length = *a.position + a.offset + 1;
  const int slice = (length + kAttnSplits - 1) / kAttnSplits;
  const int begin = split * slice;
  const int end = min(length, begin + slice);
  const int warp = tid >> 5, lane = tid & 31;
  const float scale = 1.0f / sqrtf(static_cast<float>(hd));
  for (int i = tid; i < group * hd; i += kTeamThreads) {
    s.q[i / hd][QuerySlot(i % hd, per)] = __ldcg(a.queries + (kh * group) * hd + i);
  }
  sync();
  float m[kMaxGroup], l[kMaxGroup], acc[kMaxGroup][kMaxPerLane];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      acc[g][i] = 0.f;
    }
  }
  const int kv = a.kv_heads * hd;
  // Two positions per pass, their four loads in flight together.
  for (int j0 = begin + 2 * warp; j0 < end; j0 += 2 * kTeamWarps) {
    float kf[2][kMaxPerLane], vf[2][kMaxPerLane];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int j = min(j0 + u, end - 1);
      const __half* key = a.keys + static_cast<size_t>(j) * kv + kh * hd + lane * per;
      const __half* val = a.values + static_cast<size_t>(j) * kv + kh * hd + lane * per;
      LoadHalves(key, per, kf[u]);
      LoadHalves(val, per, vf[u]);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (j0 + u < end) {
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
          if (g < group) {
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < kMaxPerLane; ++i) {
              if (i < per) {
                dot = fmaf(s.q[g][i * 32 + lane], kf[u][i], dot);
              }
            }
            const float sc = WarpSum(dot) * scale;
            const float m_new = fmaxf(m[g], sc);
            const float keep = expf(m[g] - m_new);   // 0 on the first position
            const float p = expf(sc - m_new);
            l[g] = l[g] * keep + p;
#pragma unroll
            for (int i = 0; i < kMaxPerLane; ++i) {
              acc[g][i] = acc[g][i] * keep + p * vf[u][i];
            }
            m[g] = m_new;
          }
        }
      }
    }
  }
  // Merge the warps, one query head at a time.
  for (int g = 0; g < group; ++g) {
    float mg = -INFINITY, lg = 0.f, ag[kMaxPerLane];
#pragma unroll
    for (int gg = 0; gg < kMaxGroup; ++gg) {
      if (gg == g) {
        mg = m[gg];
        lg = l[gg];
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
          ag[i] = acc[gg][i];
        }
      }
    }
    sync();
    if (lane == 0) {
      s.merge_m[warp] = mg;
    }
    sync();
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kTeamWarps; ++w) {
      top = fmaxf(top, s.merge_m[w]);
    }
    const float wgt = mg == -INFINITY ? 0.f : expf(mg - top);
    if (lane == 0) {
      s.merge_l[warp] = lg * wgt;
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      if (i < per) {
        s.merge_acc[warp][lane * per + i] = ag[i] * wgt;
      }
    }
    sync();
    float* out = a.partials + ((static_cast<size_t>(kh) * kAttnSplits + split) * group + g) * (hd + 2);
    for (int e = tid; e < hd; e += kTeamThreads) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kTeamWarps; ++w) {
        total += s.merge_acc[w][e];
      }
      out[e] = total;
    }
    if (tid == 0) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kTeamWarps; ++w) {
        total += s.merge_l[w];
      }
      out[hd] = top;
      out[hd + 1] = total;
    }
  }
  sync();   // the scratch may be reused by the team's next item
}

// Merges the slices of query head `qh` and applies the output gate
// (decoder.cpp:383-411). Two rounds of loads: the slices' maxima and sums, a
// lane each, then every thread's kAttnSplits values per output at once.
__device__ __forceinline__ void AttnMergeBody(const AttnArgs& a, int qh, int tid) {
  static_assert(kAttnSplits == 32, "a warp holds the slices, a lane each");
  const int hd = a.head_dim;
  const int group = a.heads / a.kv_heads;
  const int kh = qh / group, g = qh % group;
  const int lane = tid & 31;
  auto slice = [&](int s) {
    return a.partials + ((static_cast<size_t>(kh) * kAttnSplits + s) * group + g) * (hd + 2);
  };
  // Every warp works the weights out for itself (no shared memory, no barrier).
  const float m = __ldcg(slice(lane) + hd);
  const float l = __ldcg(slice(lane) + hd + 1);
  float top = m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    top = fmaxf(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
  }
  const float mine = m == -INFINITY ? 0.f : expf(m - top);
  float total = 0.f;   // in slice order
  float wgt[kAttnSplits];
#pragma unroll
  for (int s = 0; s < kAttnSplits; ++s) {
    wgt[s] = __shfl_sync(0xFFFFFFFFu, mine, s);
    total += __shfl_sync(0xFFFFFFFFu, mine * l, s);
  }
  const float inv_total = 1.0f / total;
  const float* gate = a.in + static_cast<size_t>(qh) * 2 * hd + hd;
  for (int e = tid; e < hd; e += kTeamThreads) {
    float part[kAttnSplits];
#pragma unroll
    for (int s = 0; s < kAttnSplits; ++s) {
      part[s] = __ldcg(slice(s) + e);
    }
    const float gv = __ldcg(gate + e);
    float out = 0.f;
#pragma unroll
    for (int s = 0; s < kAttnSplits; ++s) {
      out += wgt[s] * part[s];
    }
    a.ctx[qh * hd + e] = out * (inv_total * SigmoidDev(gv));
  }
}

}  // namespace gufo
