/* CPU oracle for the decode hot path: TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU arithmetic for the GGUF K-quant
 * dequantization, the fused row dots, the stacked-parts matrix product, the
 * Gated DeltaNet decode step and the MoE routing. Nothing in the product
 * library links or calls this file: only the tests, the smoke check and the
 * benchmark's cpu_baseline leg do, and only as the checker.
 *
 * Each function names the reference file:line it follows (paths are relative
 * to the reference project's root).
 */
#ifndef GUFO_ORACLE_H_
#define GUFO_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids (src/core/gguf.hpp:16-24). */
enum {
  GUFO_ORACLE_F32 = 0,
  GUFO_ORACLE_F16 = 1,
  GUFO_ORACLE_Q8_0 = 8,
  GUFO_ORACLE_Q4_K = 12,
  GUFO_ORACLE_Q5_K = 13,
  GUFO_ORACLE_Q6_K = 14,
  GUFO_ORACLE_BF16 = 30,
};

/* src/core/quant.cpp:129-155 */
float gufo_oracle_half_to_float(uint16_t h);
/* src/core/quant.cpp:158-167 */
void gufo_oracle_scale_min_k4(size_t j, const uint8_t* q, uint8_t* scale,
                              uint8_t* min);
/* src/core/quant.cpp:183-219; 0 for an unknown type. */
size_t gufo_oracle_block_elements(int type);
size_t gufo_oracle_block_bytes(int type);
size_t gufo_oracle_row_bytes(int type, size_t n);
/* src/core/quant.cpp:221-260. Returns 0, or -1 for an unknown type or a
 * partial block. */
int gufo_oracle_dequantize(int type, const uint8_t* src, float* dst, size_t n);

/* One row dotted with fp32 x, fp32 accumulation in the lane order of the
 * reference's AVX2 bodies (src/models/qwen35/gguf_dot.hpp:31-69, 115-188,
 * 203-290; F32 rows: src/core/vec.hpp:18-52), so results are bit-identical
 * with the reference built with -march=x86-64-v3. NaN for an unknown type. */
float gufo_oracle_dot(int type, const uint8_t* row, const float* x, size_t n);
/* The same row in the reference's Precision::kDouble arithmetic: dequantize,
 * then a double sum (src/models/qwen35/gguf_projections.cpp:48-54,277-283). */
float gufo_oracle_dot_double(int type, const uint8_t* row, const float* x,
                             size_t n);

/* Rows [first, first + rows) of a row-major matrix of `type` whose rows hold
 * `cols` values (src/models/qwen35/gguf_projections.hpp:40-44). */
typedef struct {
  const uint8_t* data;
  int type;
  size_t first;
  size_t rows;
} gufo_oracle_rows;

/* y[t] = [W_0 x[t] | W_1 x[t] | ...] for `tokens` rows of `cols` inputs
 * (src/models/qwen35/gguf_projections.cpp:239-286). `exact` selects the
 * double-precision dots. Single-threaded; every output is one dot product. */
int gufo_oracle_matmul(const gufo_oracle_rows* parts, int nparts, size_t cols,
                       const float* x, int tokens, float* y, int exact);

/* The delta rule of one value head on a dk x dk state S[i (key)][j (value)]
 * (src/models/qwen35/decoder.cpp:234-257): u = (decay S)^T k,
 * delta = beta (v - u), S' = decay S + k delta^T, y = S'^T q. `dst` may equal
 * `src`. q and k are already normalised; `beta` and `decay` are the gate
 * values themselves. Fused multiply-adds as the reference's build emits them
 * (src/models/qwen35_2b/deltanet.cpp:93-97). */
void gufo_oracle_delta_rule(const float* src, float* dst, int dk,
                            const float* k, const float* q, const float* v,
                            float decay, float beta, float* y);

/* Small weights of one Gated DeltaNet layer (src/models/qwen35/decoder.cpp:
 * 40-47): conv [channels][kernel], ssm_a, dt_bias [value heads], ssm_norm [dk]. */
typedef struct {
  int key_heads;
  int value_heads;
  int head_dim;
  int conv_kernel;
  float rms_eps;
  const float* conv;
  const float* ssm_a;
  const float* dt_bias;
  const float* ssm_norm;
} gufo_oracle_deltanet_layer;

/* Mixer::Linear (src/models/qwen35/decoder.cpp:161-265): `in` is
 * [qkv (2 key_dim + value_dim) | z (value_dim) | alpha | beta (value heads)];
 * conv_state [kernel - 1][channels] advances in place; ssm [heads][dk][dk] is
 * updated in place or, with ssm_out, written there; y gets value_dim values. */
void gufo_oracle_deltanet_linear(const gufo_oracle_deltanet_layer* layer,
                                 const float* in, float* conv_state,
                                 float* ssm, float* y, float* ssm_out);

/* src/models/qwen35/moe.cpp:16-47 */
void gufo_oracle_route(const float* logits, int experts, int k, int* chosen,
                       float* weights);
float gufo_oracle_shared_expert_scale(float logit);

/* out = RMS(x) * w (src/core/vec.hpp:57-63). */
void gufo_oracle_rms_norm(const float* x, const float* w, int n, float eps,
                          float* out);

#ifdef __cplusplus
}
#endif
#endif /* GUFO_ORACLE_H_ */
