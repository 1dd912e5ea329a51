// Bit-exact dequantization of GGUF Q4_K and Q6_K rows to fp32
// (quant::Dequantize, src/core/quant.cpp:33-59 and 98-125 in the reference),
// and of the other formats real files carry: Q8_0 (:21-30), Q5_K (:61-95), F16
// and BF16.
//
// HBM-bound on the fp32 writes (4 bytes out per 0.56 / 0.82 bytes in). Each
// product below is exact in fp32 (d: 11 significant bits, 6- or 7-bit scale,
// 4- or 6-bit code), so the only rounding is Q4_K's final subtraction, as on
// the CPU; the intrinsics keep the compiler from reassociating.
#include "common.cuh"

namespace gufo {
namespace {

// One thread per 32-bit word of a block's 128 nibble bytes: bytes 4c..4c+3 of
// pair p give values 4c..4c+3 of sub-block 2p (low nibbles) and 2p+1 (high).
__global__ void __launch_bounds__(256)
DequantQ4K(const uint8_t* __restrict__ src, float* __restrict__ dst,
           int64_t blocks) {
  const int64_t items = blocks * 32;
  for (int64_t item = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
       item < items; item += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = item >> 5;
    const int word = static_cast<int>(item & 31);
    const int p = word >> 3;
    const int c = word & 7;
    const uint32_t* block = reinterpret_cast<const uint32_t*>(src + b * kQ4KBytes);
    const uint32_t dd = __ldg(block);
    const float d = HalfBitsToFloat(static_cast<uint16_t>(dd & 0xFFFF));
    const float dmin = HalfBitsToFloat(static_cast<uint16_t>(dd >> 16));
    const uint32_t s0 = __ldg(block + 1), s1 = __ldg(block + 2), s2 = __ldg(block + 3);
    int sc_lo, m_lo, sc_hi, m_hi;
    ScaleMinK4(2 * p, s0, s1, s2, &sc_lo, &m_lo);
    ScaleMinK4(2 * p + 1, s0, s1, s2, &sc_hi, &m_hi);
    const float d1 = __fmul_rn(d, static_cast<float>(sc_lo));
    const float m1 = __fmul_rn(dmin, static_cast<float>(m_lo));
    const float d2 = __fmul_rn(d, static_cast<float>(sc_hi));
    const float m2 = __fmul_rn(dmin, static_cast<float>(m_hi));
    const uint32_t q = __ldg(block + 4 + word);
    float4 lo, hi;
    lo.x = __fsub_rn(__fmul_rn(d1, static_cast<float>(q & 0xF)), m1);
    lo.y = __fsub_rn(__fmul_rn(d1, static_cast<float>((q >> 8) & 0xF)), m1);
    lo.z = __fsub_rn(__fmul_rn(d1, static_cast<float>((q >> 16) & 0xF)), m1);
    lo.w = __fsub_rn(__fmul_rn(d1, static_cast<float>((q >> 24) & 0xF)), m1);
    hi.x = __fsub_rn(__fmul_rn(d2, static_cast<float>((q >> 4) & 0xF)), m2);
    hi.y = __fsub_rn(__fmul_rn(d2, static_cast<float>((q >> 12) & 0xF)), m2);
    hi.z = __fsub_rn(__fmul_rn(d2, static_cast<float>((q >> 20) & 0xF)), m2);
    hi.w = __fsub_rn(__fmul_rn(d2, static_cast<float>(q >> 28)), m2);
    float* out = dst + b * kSuperBlock + 64 * p + 4 * c;
    *reinterpret_cast<float4*>(out) = lo;
    *reinterpret_cast<float4*>(out + 32) = hi;
  }
}

// One thread per (row, block, half, l): values l, l+32, l+64, l+96 of the
// half, read from the planar device arrangement of the row.
__global__ void __launch_bounds__(256)
DequantQ6K(const uint8_t* __restrict__ src, float* __restrict__ dst,
           int64_t rows, int blocks, size_t row_bytes) {
  const int64_t items = rows * blocks * 64;
  for (int64_t item = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
       item < items; item += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t rb = item >> 6;
    const int64_t r = rb / blocks;
    const int b = static_cast<int>(rb - r * blocks);
    const int half = static_cast<int>((item >> 5) & 1);
    const int l = static_cast<int>(item & 31);
    const Q6KBlock block = Q6KBlockAt(src + r * row_bytes, blocks, b);
    const uint8_t* ql = block.ql + 64 * half;
    const uint8_t* qh = block.qh + 32 * half;
    const int8_t* sc = block.sc + 8 * half + (l >> 4);
    const float d = HalfBitsToFloat(*reinterpret_cast<const uint16_t*>(block.d));
    const int a = ql[l], c = ql[l + 32], h = qh[l];
    const int q1 = ((a & 0xF) | ((h & 3) << 4)) - 32;
    const int q2 = ((c & 0xF) | (((h >> 2) & 3) << 4)) - 32;
    const int q3 = ((a >> 4) | (((h >> 4) & 3) << 4)) - 32;
    const int q4 = ((c >> 4) | (((h >> 6) & 3) << 4)) - 32;
    float* out = dst + rb * kSuperBlock + 128 * half + l;
    out[0] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[0])), static_cast<float>(q1));
    out[32] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[2])), static_cast<float>(q2));
    out[64] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[4])), static_cast<float>(q3));
    out[96] = __fmul_rn(__fmul_rn(d, static_cast<float>(sc[6])), static_cast<float>(q4));
  }
}

// One thread per value: w = d * q (DequantQ8_0, quant.cpp:21-30). Blocks are
// 34 bytes, so the scale sits on a 2-byte boundary.
__global__ void __launch_bounds__(256)
DequantQ8_0(const uint8_t* __restrict__ src, float* __restrict__ dst, int64_t values) {
  for (int64_t item = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; item < values;
       item += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint8_t* block = src + (item >> 5) * kQ8Bytes;
    const float d = HalfBitsToFloat(*reinterpret_cast<const uint16_t*>(block));
    const int q = static_cast<int8_t>(block[2 + (item & 31)]);
    dst[item] = __fmul_rn(d, static_cast<float>(q));
  }
}

// One thread per (block, sub-block pair p, l): values l of sub-blocks 2p and
// 2p + 1; the fifth bit of a code is bit 2p / 2p + 1 of qh[l] (DequantQ5_K,
// quant.cpp:61-95).
__global__ void __launch_bounds__(256)
DequantQ5K(const uint8_t* __restrict__ src, float* __restrict__ dst, int64_t blocks) {
  const int64_t items = blocks * 128;
  for (int64_t item = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; item < items;
       item += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = item >> 7;
    const int p = static_cast<int>((item >> 5) & 3);
    const int l = static_cast<int>(item & 31);
    const uint8_t* bytes = src + b * kQ5KBytes;
    const uint32_t* block = reinterpret_cast<const uint32_t*>(bytes);
    const uint32_t dd = __ldg(block);
    const float d = HalfBitsToFloat(static_cast<uint16_t>(dd & 0xFFFF));
    const float dmin = HalfBitsToFloat(static_cast<uint16_t>(dd >> 16));
    int sc_lo, m_lo, sc_hi, m_hi;
    ScaleMinK4(2 * p, __ldg(block + 1), __ldg(block + 2), __ldg(block + 3), &sc_lo, &m_lo);
    ScaleMinK4(2 * p + 1, __ldg(block + 1), __ldg(block + 2), __ldg(block + 3), &sc_hi, &m_hi);
    const int h = bytes[16 + l];
    const int a = bytes[48 + 32 * p + l];
    const int lo = (a & 0xF) + (((h >> (2 * p)) & 1) << 4);
    const int hi = (a >> 4) + (((h >> (2 * p + 1)) & 1) << 4);
    float* out = dst + b * kSuperBlock + 64 * p + l;
    out[0] = __fsub_rn(__fmul_rn(__fmul_rn(d, static_cast<float>(sc_lo)), static_cast<float>(lo)),
                       __fmul_rn(dmin, static_cast<float>(m_lo)));
    out[32] = __fsub_rn(__fmul_rn(__fmul_rn(d, static_cast<float>(sc_hi)), static_cast<float>(hi)),
                        __fmul_rn(dmin, static_cast<float>(m_hi)));
  }
}

// fp16 or bf16 values to fp32.
__global__ void __launch_bounds__(256)
DequantHalf(const uint16_t* __restrict__ src, float* __restrict__ dst, int64_t values, int bf16) {
  for (int64_t item = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; item < values;
       item += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint16_t bits = src[item];
    float value;
    if (bf16) {
      value = __uint_as_float(static_cast<uint32_t>(bits) << 16);
    } else if ((bits & 0x7C00u) == 0x7C00u) {
      // Infinities and NaNs keep their payload as quant::HalfToFloat does
      // (src/core/quant.cpp:148-149); the hardware conversion would quiet them.
      value = __uint_as_float((static_cast<uint32_t>(bits & 0x8000u) << 16) | 0x7F800000u |
                              (static_cast<uint32_t>(bits & 0x3FFu) << 13));
    } else {
      value = HalfBitsToFloat(bits);
    }
    dst[item] = value;
  }
}

}  // namespace
}  // namespace gufo

using gufo::Fail;

extern "C" {

int gufo_cuda_dequantize_device(gufo_cuda_ctx* ctx, gufo_cuda_matrix matrix,
                                int64_t first, int64_t rows, float* device_dst) {
  if (ctx == nullptr || device_dst == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "dequantize: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  const gufo::Matrix* m = ctx->FindMatrix(matrix);
  if (m == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "dequantize: unknown matrix handle");
  }
  if (first < 0 || rows < 0 || first + rows > m->rows) {
    return Fail(GUFO_CUDA_SHAPE, "dequantize: rows out of range");
  }
  if (rows == 0) {
    return GUFO_CUDA_OK;
  }
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  const uint8_t* src = m->data + static_cast<size_t>(first) * m->row_bytes;
  const int64_t values = rows * m->cols;
  if (m->type == GUFO_CUDA_F32) {
    GUFO_CUDA_TRY(cudaMemcpyAsync(device_dst, src, static_cast<size_t>(values) * 4,
                                  cudaMemcpyDeviceToDevice, ctx->stream));
    return GUFO_CUDA_OK;
  }
  const int64_t blocks = values / gufo::kSuperBlock;
  const int64_t items = m->type == GUFO_CUDA_Q4_K   ? blocks * 32
                        : m->type == GUFO_CUDA_Q6_K ? blocks * 64
                        : m->type == GUFO_CUDA_Q5_K ? blocks * 128
                                                    : values;
  const int64_t want = (items + 255) / 256;
  const int grid = static_cast<int>(want < ctx->sm_count * 8 ? want : ctx->sm_count * 8);
  if (m->type == GUFO_CUDA_Q4_K) {
    gufo::DequantQ4K<<<grid, 256, 0, ctx->stream>>>(src, device_dst, blocks);
  } else if (m->type == GUFO_CUDA_Q5_K) {
    gufo::DequantQ5K<<<grid, 256, 0, ctx->stream>>>(src, device_dst, blocks);
  } else if (m->type == GUFO_CUDA_Q8_0) {
    gufo::DequantQ8_0<<<grid, 256, 0, ctx->stream>>>(src, device_dst, values);
  } else if (m->type == GUFO_CUDA_F16 || m->type == GUFO_CUDA_BF16) {
    gufo::DequantHalf<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const uint16_t*>(src), device_dst, values,
                                                     m->type == GUFO_CUDA_BF16 ? 1 : 0);
  } else {
    gufo::DequantQ6K<<<grid, 256, 0, ctx->stream>>>(src, device_dst, rows,
                                                     static_cast<int>(m->cols / gufo::kSuperBlock), m->row_bytes);
  }
  ctx->launches.fetch_add(1);
  GUFO_CUDA_TRY(cudaGetLastError());
  return GUFO_CUDA_OK;
}

int gufo_cuda_dequantize(gufo_cuda_ctx* ctx, gufo_cuda_matrix matrix,
                         int64_t first, int64_t rows, float* host_dst) {
  if (ctx == nullptr || host_dst == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "dequantize: null pointer");
  }
  int64_t cols = 0;
  {
    std::lock_guard<std::mutex> lock(ctx->mu);
    const gufo::Matrix* m = ctx->FindMatrix(matrix);
    if (m == nullptr) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "dequantize: unknown matrix handle");
    }
    if (first < 0 || rows < 0 || first + rows > m->rows) {
      return Fail(GUFO_CUDA_SHAPE, "dequantize: rows out of range");
    }
    cols = m->cols;
    const size_t bytes = static_cast<size_t>(rows) * cols * 4;
    if (bytes == 0) {
      return GUFO_CUDA_OK;
    }
    int rc = ctx->Reserve(&ctx->stage_y, &ctx->stage_y_bytes, bytes);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
  }
  int rc = gufo_cuda_dequantize_device(ctx, matrix, first, rows, ctx->stage_y);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  return gufo_cuda_download(ctx, host_dst, ctx->stage_y,
                            static_cast<size_t>(rows) * cols * 4);
}

}  // extern "C"
