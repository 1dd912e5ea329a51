/* CPU oracle for the decode hot path: TEST INFRASTRUCTURE ONLY (see
 * gufo_oracle.h). Plain C; build with -ffp-contract=off so that the only fused
 * multiply-adds are the fmaf() calls written below, which sit where the
 * reference's AVX2 intrinsics, or its compiler at -O3 -march=x86-64-v3, fuse.
 *
 * Parity is pinned: the tests check this file against the reference's golden
 * dequantization fixtures and, bit for bit, against the reference's own
 * sources compiled into oracle/_ref.
 */
#include "gufo_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

enum { kSuper = 256, kSub = 32, kLanes = 8 };

static uint16_t load_u16(const uint8_t* p) {
  uint16_t v;
  memcpy(&v, p, sizeof(v));
  return v;
}

/* src/core/quant.cpp:129-155 */
float gufo_oracle_half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 0x1Fu;
  uint32_t m = h & 0x3FFu;
  uint32_t bits;
  if (e == 0x1F) {
    bits = sign | 0x7F800000u | (m << 13);
  } else if (e != 0) {
    bits = sign | ((e + 112u) << 23) | (m << 13);
  } else if (m == 0) {
    bits = sign;
  } else {
    /* Subnormal half: shift the leading one up to bit 10. */
    uint32_t exp32 = 113u;
    while ((m & 0x400u) == 0) {
      m <<= 1;
      --exp32;
    }
    bits = sign | (exp32 << 23) | ((m & 0x3FFu) << 13);
  }
  float f;
  memcpy(&f, &bits, sizeof(f));
  return f;
}

static float bf16_to_float(uint16_t h) {
  const uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, sizeof(f));
  return f;
}

/* src/core/quant.cpp:158-167 */
void gufo_oracle_scale_min_k4(size_t j, const uint8_t* q, uint8_t* scale,
                              uint8_t* min) {
  if (j < 4) {
    *scale = q[j] & 63;
    *min = q[j + 4] & 63;
    return;
  }
  *scale = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
  *min = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
}

size_t gufo_oracle_block_elements(int type) {
  switch (type) {
    case GUFO_ORACLE_F32:
    case GUFO_ORACLE_F16:
    case GUFO_ORACLE_BF16:
      return 1;
    case GUFO_ORACLE_Q8_0:
      return 32;
    case GUFO_ORACLE_Q4_K:
    case GUFO_ORACLE_Q5_K:
    case GUFO_ORACLE_Q6_K:
      return kSuper;
    default:
      return 0;
  }
}

size_t gufo_oracle_block_bytes(int type) {
  switch (type) {
    case GUFO_ORACLE_F32:
      return 4;
    case GUFO_ORACLE_F16:
    case GUFO_ORACLE_BF16:
      return 2;
    case GUFO_ORACLE_Q8_0:
      return 34;
    case GUFO_ORACLE_Q4_K:
      return 144;
    case GUFO_ORACLE_Q5_K:
      return 176;
    case GUFO_ORACLE_Q6_K:
      return 210;
    default:
      return 0;
  }
}

size_t gufo_oracle_row_bytes(int type, size_t n) {
  const size_t block = gufo_oracle_block_elements(type);
  if (block == 0 || n % block != 0) {
    return 0;
  }
  return n / block * gufo_oracle_block_bytes(type);
}

/* The K4 family's per-sub-block scale d*sc_j and offset dmin*m_j
 * (src/models/qwen35/gguf_dot.hpp:80-89). */
static void k4_scales(const uint8_t* block, float* scale, float* offset) {
  const float d = gufo_oracle_half_to_float(load_u16(block));
  const float dmin = gufo_oracle_half_to_float(load_u16(block + 2));
  for (size_t j = 0; j < 8; ++j) {
    uint8_t sc, m;
    gufo_oracle_scale_min_k4(j, block + 4, &sc, &m);
    scale[j] = d * (float)sc;
    offset[j] = dmin * (float)m;
  }
}

/* Code of value l (0..31) of sub-block j (0..7) of a Q4_K / Q5_K block. */
static int k4_code(const uint8_t* qs, const uint8_t* qh, size_t j, size_t l) {
  const uint8_t byte = qs[32 * (j / 2) + l];
  int code = (j & 1) ? byte >> 4 : byte & 0x0F;
  if (qh != NULL && ((qh[l] >> j) & 1)) {
    code += 16;
  }
  return code;
}

/* Code minus 32 of value p (0..127) of one half of a Q6_K block: ql is the
 * half's 64 low-nibble bytes, qh its 32 high-bit bytes
 * (src/core/quant.cpp:98-125). */
static int q6_code(const uint8_t* ql, const uint8_t* qh, size_t p) {
  const size_t k = p / 32;
  const size_t l = p % 32;
  const uint8_t byte = ql[l + 32 * (k & 1)];
  const int low = k < 2 ? byte & 0x0F : byte >> 4;
  const int high = (qh[l] >> (2 * k)) & 3;
  return (low | (high << 4)) - 32;
}

/* src/core/quant.cpp:22-125, 221-260 */
int gufo_oracle_dequantize(int type, const uint8_t* src, float* dst, size_t n) {
  const size_t per = gufo_oracle_block_elements(type);
  if (per == 0 || n % per != 0) {
    return -1;
  }
  const size_t blocks = n / per;
  switch (type) {
    case GUFO_ORACLE_F32:
      memcpy(dst, src, n * sizeof(float));
      return 0;
    case GUFO_ORACLE_F16:
      for (size_t i = 0; i < n; ++i) {
        dst[i] = gufo_oracle_half_to_float(load_u16(src + 2 * i));
      }
      return 0;
    case GUFO_ORACLE_BF16:
      for (size_t i = 0; i < n; ++i) {
        dst[i] = bf16_to_float(load_u16(src + 2 * i));
      }
      return 0;
    case GUFO_ORACLE_Q8_0:
      for (size_t b = 0; b < blocks; ++b, src += 34, dst += 32) {
        const float d = gufo_oracle_half_to_float(load_u16(src));
        for (size_t l = 0; l < 32; ++l) {
          dst[l] = d * (float)(int8_t)src[2 + l];
        }
      }
      return 0;
    case GUFO_ORACLE_Q4_K:
    case GUFO_ORACLE_Q5_K: {
      const int fifth = type == GUFO_ORACLE_Q5_K;
      const size_t bytes = fifth ? 176 : 144;
      for (size_t b = 0; b < blocks; ++b, src += bytes, dst += kSuper) {
        float scale[8], offset[8];
        k4_scales(src, scale, offset);
        const uint8_t* qh = fifth ? src + 16 : NULL;
        const uint8_t* qs = src + 16 + (fifth ? 32 : 0);
        for (size_t j = 0; j < 8; ++j) {
          for (size_t l = 0; l < kSub; ++l) {
            /* scale * code is exact in fp32 (11 + 6 + 5 bits), so only the
             * subtraction rounds, fused or not. */
            dst[kSub * j + l] =
                scale[j] * (float)k4_code(qs, qh, j, l) - offset[j];
          }
        }
      }
      return 0;
    }
    case GUFO_ORACLE_Q6_K:
      for (size_t b = 0; b < blocks; ++b, src += 210, dst += kSuper) {
        const int8_t* sc = (const int8_t*)(src + 192);
        const float d = gufo_oracle_half_to_float(load_u16(src + 208));
        for (size_t half = 0; half < 2; ++half) {
          const uint8_t* ql = src + 64 * half;
          const uint8_t* qh = src + 128 + 32 * half;
          for (size_t p = 0; p < 128; ++p) {
            const float ds = d * (float)sc[8 * half + p / 16];
            dst[128 * half + p] = ds * (float)q6_code(ql, qh, p);
          }
        }
      }
      return 0;
    default:
      return -1;
  }
}

/* Lanes 0..7 summed as the reference's HorizontalSum does
 * (src/models/qwen35/gguf_dot.hpp:23-28): (l + l+4), then (+2), then (+1). */
static float lane_sum(const float* v) {
  const float s0 = v[0] + v[4];
  const float s1 = v[1] + v[5];
  const float s2 = v[2] + v[6];
  const float s3 = v[3] + v[7];
  return (s0 + s2) + (s1 + s3);
}

/* src/core/vec.hpp:18-52 (AVX2 body): two sets of 8 lanes over 16 values per
 * step, added, halves added, then two horizontal adds. */
static float dot_f32(const float* a, const float* b, size_t n) {
  float acc0[kLanes] = {0}, acc1[kLanes] = {0};
  size_t i = 0;
  for (; i + 16 <= n; i += 16) {
    for (size_t l = 0; l < kLanes; ++l) {
      acc0[l] = fmaf(a[i + l], b[i + l], acc0[l]);
      acc1[l] = fmaf(a[i + 8 + l], b[i + 8 + l], acc1[l]);
    }
  }
  float s[4];
  for (size_t l = 0; l < 4; ++l) {
    s[l] = (acc0[l] + acc1[l]) + (acc0[l + 4] + acc1[l + 4]);
  }
  float total = (s[0] + s[1]) + (s[2] + s[3]);
  for (; i < n; ++i) {
    total = fmaf(a[i], b[i], total);
  }
  return total;
}

/* src/models/qwen35/gguf_dot.hpp:31-69 */
static float dot_q8_0(const uint8_t* row, const float* x, size_t n) {
  float acc[kLanes] = {0};
  for (size_t b = 0; b < n / 32; ++b, row += 34, x += 32) {
    const float d = gufo_oracle_half_to_float(load_u16(row));
    const int8_t* q = (const int8_t*)(row + 2);
    float block[kLanes] = {0};
    for (size_t step = 0; step < 4; ++step) {
      for (size_t l = 0; l < kLanes; ++l) {
        block[l] = fmaf((float)q[8 * step + l], x[8 * step + l], block[l]);
      }
    }
    for (size_t l = 0; l < kLanes; ++l) {
      acc[l] = fmaf(d, block[l], acc[l]);
    }
  }
  return lane_sum(acc);
}

/* src/models/qwen35/gguf_dot.hpp:94-106, 115-155: lane l of the accumulator
 * takes values l, l + 8, l + 16, l + 24 of every sub-block in turn, each as
 * fma(fma(code, scale, -offset), x, acc). */
static float dot_k4(const uint8_t* row, const float* x, size_t n, int fifth) {
  const size_t bytes = fifth ? 176 : 144;
  float acc[kLanes] = {0};
  for (size_t b = 0; b < n / kSuper; ++b, row += bytes, x += kSuper) {
    float scale[8], offset[8];
    k4_scales(row, scale, offset);
    const uint8_t* qh = fifth ? row + 16 : NULL;
    const uint8_t* qs = row + 16 + (fifth ? 32 : 0);
    for (size_t j = 0; j < 8; ++j) {
      for (size_t step = 0; step < 4; ++step) {
        for (size_t l = 0; l < kLanes; ++l) {
          const size_t at = 8 * step + l;
          const float w =
              fmaf((float)k4_code(qs, qh, j, at), scale[j], -offset[j]);
          acc[l] = fmaf(w, x[kSub * j + at], acc[l]);
        }
      }
    }
  }
  return lane_sum(acc);
}

/* src/models/qwen35/gguf_dot.hpp:203-258: per group of 16 values, lane l
 * holds code[l] * x[l] then fma(code[l + 8], x[l + 8], .); the group joins the
 * block as fma(scale, group, block); the block joins the row as
 * fma(d, block, acc). */
static float dot_q6_k(const uint8_t* row, const float* x, size_t n) {
  float acc[kLanes] = {0};
  for (size_t b = 0; b < n / kSuper; ++b, row += 210, x += kSuper) {
    const int8_t* sc = (const int8_t*)(row + 192);
    const float d = gufo_oracle_half_to_float(load_u16(row + 208));
    float block[kLanes] = {0};
    for (size_t half = 0; half < 2; ++half) {
      const uint8_t* ql = row + 64 * half;
      const uint8_t* qh = row + 128 + 32 * half;
      const float* xh = x + 128 * half;
      for (size_t g = 0; g < 8; ++g) {
        const float s = (float)sc[8 * half + g];
        for (size_t l = 0; l < kLanes; ++l) {
          const size_t p = 16 * g + l;
          float group = (float)q6_code(ql, qh, p) * xh[p];
          group = fmaf((float)q6_code(ql, qh, p + 8), xh[p + 8], group);
          block[l] = fmaf(s, group, block[l]);
        }
      }
    }
    for (size_t l = 0; l < kLanes; ++l) {
      acc[l] = fmaf(d, block[l], acc[l]);
    }
  }
  return lane_sum(acc);
}

float gufo_oracle_dot(int type, const uint8_t* row, const float* x, size_t n) {
  switch (type) {
    case GUFO_ORACLE_F32:
      return dot_f32((const float*)row, x, n);
    case GUFO_ORACLE_Q8_0:
      return dot_q8_0(row, x, n);
    case GUFO_ORACLE_Q4_K:
      return dot_k4(row, x, n, 0);
    case GUFO_ORACLE_Q5_K:
      return dot_k4(row, x, n, 1);
    case GUFO_ORACLE_Q6_K:
      return dot_q6_k(row, x, n);
    default:
      return NAN;
  }
}

float gufo_oracle_dot_double(int type, const uint8_t* row, const float* x,
                             size_t n) {
  float* w = (float*)malloc(n * sizeof(float));
  if (w == NULL || gufo_oracle_dequantize(type, row, w, n) != 0) {
    free(w);
    return NAN;
  }
  double sum = 0;
  for (size_t i = 0; i < n; ++i) {
    sum += (double)w[i] * x[i];
  }
  free(w);
  return (float)sum;
}

/* src/models/qwen35/gguf_projections.cpp:239-286 */
int gufo_oracle_matmul(const gufo_oracle_rows* parts, int nparts, size_t cols,
                       const float* x, int tokens, float* y, int exact) {
  size_t stride = 0;
  for (int p = 0; p < nparts; ++p) {
    if (gufo_oracle_row_bytes(parts[p].type, cols) == 0) {
      return -1;
    }
    stride += parts[p].rows;
  }
  size_t offset = 0;
  for (int p = 0; p < nparts; ++p) {
    const size_t row_bytes = gufo_oracle_row_bytes(parts[p].type, cols);
    const int fused = !exact && parts[p].type != GUFO_ORACLE_F16 &&
                      parts[p].type != GUFO_ORACLE_BF16;
    for (size_t r = 0; r < parts[p].rows; ++r) {
      const uint8_t* row = parts[p].data + (parts[p].first + r) * row_bytes;
      for (int t = 0; t < tokens; ++t) {
        const float* xt = x + (size_t)t * cols;
        float* out = y + (size_t)t * stride + offset + r;
        if (fused) {
          *out = gufo_oracle_dot(parts[p].type, row, xt, cols);
        } else if (exact) {
          *out = gufo_oracle_dot_double(parts[p].type, row, xt, cols);
        } else {
          /* F16/BF16 rows: dequantize, then the fp32 dot. */
          float* w = (float*)malloc(cols * sizeof(float));
          if (w == NULL) {
            return -1;
          }
          gufo_oracle_dequantize(parts[p].type, row, w, cols);
          *out = dot_f32(w, xt, cols);
          free(w);
        }
      }
    }
    offset += parts[p].rows;
  }
  return 0;
}

/* src/models/qwen35/decoder.cpp:234-257 */
void gufo_oracle_delta_rule(const float* src, float* dst, int dk,
                            const float* k, const float* q, const float* v,
                            float decay, float beta, float* y) {
  float* delta = (float*)calloc((size_t)dk, sizeof(float));
  for (int i = 0; i < dk; ++i) {
    const float* row = src + (size_t)i * dk;
    const float ki = k[i] * decay;
    for (int j = 0; j < dk; ++j) {
      delta[j] = fmaf(row[j], ki, delta[j]);
    }
  }
  for (int j = 0; j < dk; ++j) {
    delta[j] = beta * (v[j] - delta[j]);
    y[j] = 0.0f;
  }
  for (int i = 0; i < dk; ++i) {
    const float* row = src + (size_t)i * dk;
    float* out = dst + (size_t)i * dk;
    for (int j = 0; j < dk; ++j) {
      const float updated = fmaf(row[j], decay, k[i] * delta[j]);
      out[j] = updated;
      y[j] = fmaf(updated, q[i], y[j]);
    }
  }
  free(delta);
}

/* src/core/vec.hpp:57-63 */
void gufo_oracle_rms_norm(const float* x, const float* w, int n, float eps,
                          float* out) {
  const float inv = 1.0f / sqrtf(dot_f32(x, x, (size_t)n) / (float)n + eps);
  for (int i = 0; i < n; ++i) {
    out[i] = x[i] * inv * w[i];
  }
}

/* src/models/qwen35/decoder.cpp:26-34 */
static float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
static float silu_f(float x) { return x * sigmoid_f(x); }
static float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

/* src/models/qwen35/decoder.cpp:161-265 */
void gufo_oracle_deltanet_linear(const gufo_oracle_deltanet_layer* layer,
                                 const float* in, float* conv_state,
                                 float* ssm, float* y, float* ssm_out) {
  const int hk = layer->key_heads;
  const int hv = layer->value_heads;
  const int dk = layer->head_dim;
  const int key_dim = hk * dk;
  const int value_dim = hv * dk;
  const int channels = 2 * key_dim + value_dim;
  const int kernel = layer->conv_kernel;
  const int window = kernel - 1;
  const float* z = in + channels;
  const float* alpha = z + value_dim;
  const float* beta = alpha + hv;

  /* Causal depthwise conv over [window previous inputs, current], SiLU. */
  float* u = (float*)malloc((size_t)channels * sizeof(float));
  for (int ch = 0; ch < channels; ++ch) {
    const float* kw = layer->conv + (size_t)ch * kernel;
    float acc = kw[window] * in[ch];
    for (int t = 0; t < window; ++t) {
      acc = fmaf(kw[t], conv_state[(size_t)t * channels + ch], acc);
    }
    u[ch] = silu_f(acc);
  }
  memmove(conv_state, conv_state + channels,
          (size_t)(window - 1) * channels * sizeof(float));
  memcpy(conv_state + (size_t)(window - 1) * channels, in,
         (size_t)channels * sizeof(float));

  /* L2-normalise q and k per key head; q also takes 1/sqrt(dk). */
  float* q = u;
  float* k = u + key_dim;
  const float* v = k + key_dim;
  const float q_scale = 1.0f / sqrtf((float)dk);
  for (int head = 0; head < hk; ++head) {
    float* qh = q + head * dk;
    float* kh = k + head * dk;
    const float q_inv = 1.0f / sqrtf(dot_f32(qh, qh, (size_t)dk) + 1e-6f);
    const float qs = q_inv * q_scale;
    for (int e = 0; e < dk; ++e) {
      qh[e] *= qs;
    }
    const float k_inv = 1.0f / sqrtf(dot_f32(kh, kh, (size_t)dk) + 1e-6f);
    for (int e = 0; e < dk; ++e) {
      kh[e] *= k_inv;
    }
  }

  for (int head = 0; head < hv; ++head) {
    const int kh = head % hk; /* value heads tile the key heads */
    const float b = sigmoid_f(beta[head]);
    const float decay = expf(
        layer->ssm_a[head] * softplus_f(alpha[head] + layer->dt_bias[head]));
    const size_t at = (size_t)head * dk * dk;
    float* yh = y + head * dk;
    gufo_oracle_delta_rule(ssm + at, (ssm_out != NULL ? ssm_out : ssm) + at, dk,
                           k + kh * dk, q + kh * dk, v + head * dk, decay, b,
                           yh);
    /* Gated RMSNorm: RMS(o) * w * silu(z). */
    gufo_oracle_rms_norm(yh, layer->ssm_norm, dk, layer->rms_eps, yh);
    for (int j = 0; j < dk; ++j) {
      yh[j] *= silu_f(z[head * dk + j]);
    }
  }
  free(u);
}

/* src/models/qwen35/moe.cpp:16-42 */
void gufo_oracle_route(const float* logits, int experts, int k, int* chosen,
                       float* weights) {
  double* prob = (double*)malloc((size_t)experts * sizeof(double));
  char* taken = (char*)calloc((size_t)experts, 1);
  float top_logit = logits[0];
  for (int e = 1; e < experts; ++e) {
    top_logit = logits[e] > top_logit ? logits[e] : top_logit;
  }
  double total = 0;
  for (int e = 0; e < experts; ++e) {
    prob[e] = exp((double)logits[e] - (double)top_logit);
    total += prob[e];
  }
  /* The k most probable, ties to the lower id, in order of probability. */
  for (int slot = 0; slot < k; ++slot) {
    int best = -1;
    for (int e = 0; e < experts; ++e) {
      if (!taken[e] && (best < 0 || prob[e] > prob[best])) {
        best = e;
      }
    }
    taken[best] = 1;
    chosen[slot] = best;
  }
  double top = 0;
  for (int slot = 0; slot < k; ++slot) {
    top += prob[chosen[slot]] / total;
  }
  if (top < 6.103515625e-5) { /* smallest normal fp16 */
    top = 6.103515625e-5;
  }
  for (int slot = 0; slot < k; ++slot) {
    weights[slot] = (float)(prob[chosen[slot]] / total / top);
  }
  free(prob);
  free(taken);
}

/* src/models/qwen35/moe.cpp:44-47 */
float gufo_oracle_shared_expert_scale(float logit) {
  return (float)(1.0 / (1.0 + exp(-(double)logit)));
}
