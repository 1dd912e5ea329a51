/* gufo_cuda.h - C ABI of the B200 (sm_100a) backend for gufo-npu's decode hot
 * path: GGUF Q4_K / Q6_K dequant-fused GEMV and small-M GEMM behind every
 * projection, bit-exact dequantization, the Gated DeltaNet decode step and the
 * routed-expert FFN of the MoE models.
 *
 * This is the boundary a `src/cuda` backend binds beside the reference's
 * `src/npu`: plain pointers and sizes, no C++ types, no exceptions. Each entry
 * point names the reference interface it stands behind (paths are relative to
 * the reference project's root).
 *
 * Conventions
 *  - Every function returns a gufo_cuda_status (0 = ok) and never throws or
 *    aborts; gufo_cuda_last_error() gives the text of the calling thread's last
 *    failure on that context.
 *  - A context belongs to one CUDA device and one stream. Calls on one context
 *    are serialised by an internal mutex, as the reference serialises products
 *    on its shared pool (src/models/qwen35/gguf_projections.cpp:253).
 *  - `_device` variants take device pointers and only enqueue work on the
 *    context's stream; the plain variants take host pointers, copy inputs up and
 *    results down, and return after the stream has drained.
 *  - All activations and outputs are fp32. Matrices are row-major GGUF blocks:
 *    `rows` rows of `cols` values, cols contiguous (ggml shape [cols, rows]).
 *  - There is no CPU fallback: without a usable device, context creation fails.
 */
#ifndef GUFO_CUDA_H_
#define GUFO_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum gufo_cuda_status {
  GUFO_CUDA_OK = 0,
  GUFO_CUDA_BAD_ARGUMENT = 1,     /* null pointer, bad count, unknown handle   */
  GUFO_CUDA_SHAPE = 2,            /* widths or row ranges that do not fit      */
  GUFO_CUDA_UNSUPPORTED_TYPE = 3, /* a ggml type this backend does not run     */
  GUFO_CUDA_RUNTIME = 4,          /* a CUDA call failed; see last_error        */
  GUFO_CUDA_OUT_OF_MEMORY = 5,
  GUFO_CUDA_TIMEOUT = 6,          /* a bounded device-side wait ran out        */
  GUFO_CUDA_TOO_LARGE = 7         /* beyond a fixed capacity of the entry point */
} gufo_cuda_status;

/* ggml tensor type ids, as in the reference's gguf::GgmlType
 * (src/core/gguf.hpp:16-24). */
enum {
  GUFO_CUDA_F32 = 0,
  GUFO_CUDA_F16 = 1,   /* dequantization only (embeddings) */
  GUFO_CUDA_Q8_0 = 8,
  GUFO_CUDA_Q4_K = 12,
  GUFO_CUDA_Q5_K = 13,
  GUFO_CUDA_Q6_K = 14,
  GUFO_CUDA_BF16 = 30  /* dequantization only */
};

typedef struct gufo_cuda_ctx gufo_cuda_ctx;
/* Opaque matrix handle (> 0). */
typedef int64_t gufo_cuda_matrix;
/* Opaque handle of one DeltaNet layer's small weights (> 0). */
typedef int64_t gufo_cuda_deltanet_layer;

/* ---- context ---------------------------------------------------------- */

/* Creates a context on CUDA device `device`. `stream` is a cudaStream_t to
 * enqueue on, or NULL for a stream the context creates and owns. Stands where
 * the reference opens its accelerator (npu::GemvRuntime, src/npu/gemv.hpp:82-
 * 100); fails with GUFO_CUDA_RUNTIME when no sm_100 device is usable, as the
 * reference's stub runtime throws (src/npu/gemv_stub.cpp:8-10). */
int gufo_cuda_ctx_create(int device, void* stream, gufo_cuda_ctx** out);
int gufo_cuda_ctx_destroy(gufo_cuda_ctx* ctx);
/* Replaces the stream later work is enqueued on (not owned). */
int gufo_cuda_ctx_set_stream(gufo_cuda_ctx* ctx, void* stream);
int gufo_cuda_ctx_synchronize(gufo_cuda_ctx* ctx);
/* Text of the last failure of a call on `ctx` (or of ctx_create when ctx is
 * NULL) made by this thread; valid until that thread's next failing call. */
const char* gufo_cuda_last_error(const gufo_cuda_ctx* ctx);
/* Tuning and test switches, by name. "general_gemv" = 1 routes every product
 * through the general (non tensor-core) kernel; 0 (default) picks per part.
 * "deltanet_early_state" = 1 is the caller's promise that the DeltaNet states
 * and conv windows it passes were not written by the kernels enqueued shortly
 * before the call (true when each is touched once per decode step; kernels
 * launch ahead of one another, so "shortly" is a handful of launches): the
 * kernels then request them ahead of their dependency on the previous kernel.
 * "tc_gemm" = 1 (default) runs products of 17 or more token rows (where the
 * GEMV kernels would need a third pass over the weights) on the tcgen05 GEMM,
 * 0 keeps them on the 8-token passes of the GEMV kernels, 2 sends every
 * product of 16 or more rows to the GEMM.
 * "gemv_variant" = 1 is a timing aid: the tensor-core GEMV kernels skip their
 * multiplies and only move the weights (outputs are then meaningless).
 * "reuse_image" = 1 is a timing aid: products skip the staging of x and
 * multiply against the previously staged activations. */
int gufo_cuda_ctx_set_option(gufo_cuda_ctx* ctx, const char* name, int value);
/* Number of kernels this context has launched so far. */
int64_t gufo_cuda_launch_count(const gufo_cuda_ctx* ctx);

/* ---- device memory (decode state lives on the device between steps) ---- */

/* Plain device buffers for activations, DeltaNet states and conv windows.
 * States are raw fp32 in the reference's layout (DecodeState::Layer,
 * src/models/qwen35/decoder.hpp:26-37), so upload/download are the checkpoint
 * and rollback primitives (src/models/qwen35/state_capture.hpp:8-14). */
int gufo_cuda_malloc(gufo_cuda_ctx* ctx, size_t bytes, void** device_ptr);
int gufo_cuda_free(gufo_cuda_ctx* ctx, void* device_ptr);
int gufo_cuda_upload(gufo_cuda_ctx* ctx, void* device_dst, const void* host_src,
                     size_t bytes);
int gufo_cuda_download(gufo_cuda_ctx* ctx, void* host_dst,
                       const void* device_src, size_t bytes);
int gufo_cuda_memset_zero(gufo_cuda_ctx* ctx, void* device_ptr, size_t bytes);

/* ---- weights ---------------------------------------------------------- */

/* Copies a GGUF tensor's rows to the device once, as the reference's NPU
 * GEMV uploads at construction (npu::Q4nxGemv, src/npu/gemv.hpp:136-144). The
 * host bytes are not referenced after the call. `cols` must be a whole number
 * of blocks of `ggml_type` (quant::RowBytes, src/core/quant.cpp:221-227).
 * Types: Q4_K, Q6_K and F32 (the alpha/beta and router rows,
 * src/models/qwen35/gguf_projections.cpp:126-131,162-170) on every path; Q8_0
 * and Q5_K (the other row formats of real UD-Q4_K_XL files,
 * src/models/qwen35/gguf_dot.hpp:31-69,190-193) for products on the general
 * kernel and dequantization; F16 and BF16 for dequantization only
 * (src/core/quant.cpp:221-260). */
int gufo_cuda_matrix_upload(gufo_cuda_ctx* ctx, int ggml_type,
                            const void* host_bytes, int64_t rows, int64_t cols,
                            gufo_cuda_matrix* out);
/* The same over bytes already on the device; they are borrowed, not copied,
 * and must outlive the handle (GgufProjections keeps pointers into the mapped
 * file the same way, src/models/qwen35/gguf_projections.hpp:28). */
int gufo_cuda_matrix_from_device(gufo_cuda_ctx* ctx, int ggml_type,
                                 const void* device_bytes, int64_t rows,
                                 int64_t cols, gufo_cuda_matrix* out);
int gufo_cuda_matrix_free(gufo_cuda_ctx* ctx, gufo_cuda_matrix matrix);

/* ---- dequantization ---------------------------------------------------- */

/* quant::Dequantize (src/core/quant.cpp:33-59 Q4_K, 98-125 Q6_K, 221-260):
 * rows [first, first + rows) of `matrix` to fp32, bit for bit the reference's
 * values. Used for embedding rows (src/models/qwen35/decoder.cpp:486-489). */
int gufo_cuda_dequantize(gufo_cuda_ctx* ctx, gufo_cuda_matrix matrix,
                         int64_t first, int64_t rows, float* host_dst);
int gufo_cuda_dequantize_device(gufo_cuda_ctx* ctx, gufo_cuda_matrix matrix,
                                int64_t first, int64_t rows, float* device_dst);

/* ---- projections ------------------------------------------------------- */

/* Rows [first, first + rows) of a matrix: GgufProjections::Rows
 * (src/models/qwen35/gguf_projections.hpp:40-44). */
typedef struct gufo_cuda_rows {
  gufo_cuda_matrix w;
  int64_t first;
  int64_t rows;
} gufo_cuda_rows;

/* GgufProjections::MatMul (src/models/qwen35/gguf_projections.cpp:239-286),
 * the product behind Projections::Apply and ApplyExpert
 * (src/models/qwen35/projections.hpp:45-59):
 *   y[t] = [W_0 x[t] | W_1 x[t] | ...]  for t in [0, tokens)
 * x is `tokens` rows of `cols` fp32 (all parts share cols), y is `tokens` rows
 * of sum(parts[p].rows) fp32. Each output is one row dot, so results do not
 * depend on how rows are stacked or how many tokens come together.
 * The _device forms only enqueue on the context's stream. Products of two or
 * more tokens stage their input in scratch memory the context owns; the first
 * product of a larger shape makes it grow (a cudaMalloc, no wait, the outgrown
 * block is kept until gufo_cuda_ctx_destroy so that CUDA graphs captured
 * earlier stay valid). A stream capture cannot allocate: while the stream is
 * being captured such a product returns GUFO_CUDA_BAD_ARGUMENT instead, so run
 * every shape once before capturing it. */
int gufo_cuda_matmul(gufo_cuda_ctx* ctx, const gufo_cuda_rows* parts,
                     int nparts, const float* host_x, int tokens, float* host_y);
int gufo_cuda_matmul_device(gufo_cuda_ctx* ctx, const gufo_cuda_rows* parts,
                            int nparts, const float* device_x, int tokens,
                            float* device_y);

/* A product with its input step fused into the GEMV kernels, for chains of
 * products that never leave the device: the options of the reference's NPU GEMV
 * (npu::Q4nxGemv::Run with npu::Prologue / npu::Epilogue, src/npu/gemv.hpp:
 * 58-68,134-152), which its NPU decoders chain per layer
 * (src/models/qwen35_2b/npu_decoder.cpp:558-628).
 *   PLAIN     x rows as they are (Prologue::kPlain).
 *   RES_NORM  x = RMSNorm(residual + delta) * norm_weight; residual + delta
 *             also goes to residual_out (Prologue::kResNorm: "H + D also goes to
 *             the residual buffer"); the normed rows land in scratch.
 *   SWIGLU    x[i] = silu(g[i]) * u[i] over rows [g | u] of 2 * cols values: the
 *             previous product's Epilogue::kSwiGlu met at this product's input
 *             (Prologue::kAct), so the stacked gate / up product stores plain rows.
 * Rows of `tokens` tokens follow one another (cols apart; 2 * cols for SWIGLU
 * inputs). All pointers are 16-byte aligned device pointers. Q4_K and Q6_K parts
 * take the fused kernels when the rows fit their shared-memory image (up to
 * eight tokens; fewer for wide rows); other parts, or more rows, read the
 * materialised rows from scratch. */
enum {
  GUFO_CUDA_PROLOGUE_PLAIN = 0,
  GUFO_CUDA_PROLOGUE_RES_NORM = 1,
  GUFO_CUDA_PROLOGUE_SWIGLU = 2
};
typedef struct gufo_cuda_fused_input {
  int prologue;
  const float* x;            /* PLAIN: [tokens][cols]; SWIGLU: [tokens][2 * cols] */
  const float* residual;     /* RES_NORM: H, [tokens][cols] */
  const float* delta;        /* RES_NORM: D, [tokens][cols] (may be NULL) */
  const float* norm_weight;  /* RES_NORM: [cols] */
  float rms_eps;
  float* residual_out;       /* RES_NORM: H + D, [tokens][cols]; not the same buffer as residual */
  float* scratch;            /* RES_NORM, SWIGLU: [tokens][cols], the product's input rows */
  int* advance;              /* RES_NORM: an int counter incremented by `tokens` (may be NULL) */
  int delta_parts;           /* RES_NORM: D is the sum, in order, of this many vectors starting at   */
  int delta_stride;          /*   delta, delta_stride floats apart (0 or 1: delta alone). More than  */
                             /*   one: partial sums of ranks that split a product over its columns;  */
                             /*   one token, Q4_K / Q6_K parts on the tensor-core GEMV only.        */
  int epilogue;              /* GUFO_CUDA_EPILOGUE_SWIGLU: the parts are an FFN's gate and up rows    */
                             /*   (two parts, equal whole 16-row tiles, one of Q4_K / Q6_K) and y    */
                             /*   receives silu(gate) * up, [tokens][rows / 2], from the product's   */
                             /*   own kernel (npu::Epilogue::kSwiGlu, src/npu/gemv.hpp:64-68). Where  */
                             /*   the kernel cannot (more tile pairs than resident thread blocks,    */
                             /*   other formats) the call returns GUFO_CUDA_UNSUPPORTED_TYPE and      */
                             /*   enqueues nothing: ask for plain rows and a SWIGLU input instead.   */
} gufo_cuda_fused_input;
enum { GUFO_CUDA_EPILOGUE_NONE = 0, GUFO_CUDA_EPILOGUE_SWIGLU = 1 };
int gufo_cuda_matmul_fused_device(gufo_cuda_ctx* ctx, const gufo_cuda_rows* parts,
                                  int nparts, const gufo_cuda_fused_input* input,
                                  int tokens, float* device_y);

/* The Q4_K product for callers that must not allocate device memory while
 * they run: code inside a region where cudaMalloc is off limits (a stream that
 * is being captured, a latency-critical loop) or a host that has handed the
 * whole device to its own arena and plans every byte up front. It has no
 * counterpart in the reference. The weights are plain GGUF Q4_K bytes the
 * caller already holds on the device (`rows` rows of `cols` values, 16-byte
 * aligned); x is `tokens` (1..8) rows of `cols` fp32, y `tokens` rows of `rows`
 * fp32, both on the device. The fixed-point copy of x that the tensor-core
 * kernel multiplies against goes into a 64 KiB buffer built into the library
 * (every GPU that loads the library holds those 64 KiB until the process ends)
 * instead of the context's growable buffer, and the call performs no
 * cudaMalloc, cudaFree or other allocating call. Shapes whose staged
 * activations exceed the 64 KiB (3 * tokens * (cols + 32) + tokens * cols / 8 +
 * cols / 8 bytes, roughly) return GUFO_CUDA_TOO_LARGE.
 * The first call on a device looks up the buffer's address; make that call
 * before any stream capture begins. All calls share the one buffer: calls that
 * can overlap on the GPU (different streams or contexts) race on it. Nothing
 * in it needs clearing between calls; each call rewrites what it reads. */
int gufo_cuda_matmul_q4k_static_device(gufo_cuda_ctx* ctx,
                                       const void* device_weights, int64_t rows,
                                       int64_t cols, const float* device_x,
                                       int tokens, float* device_y);

/* ---- Gated DeltaNet decode step ---------------------------------------- */

/* One sequence's inputs to the delta rule with the gates already evaluated
 * (the arithmetic of src/models/qwen35/decoder.cpp:234-257 per value head):
 *   u = (decay S)^T k; delta = beta (v - u); S' = decay S + k delta^T; y = S'^T q
 * `state` is [value_heads][head_dim (key i)][head_dim (value j)] fp32 on the
 * device. With `state_out` the new state goes there and `state` is left
 * unchanged (a draft token that may be rolled back: the ssm_out argument of
 * Mixer::Linear, src/models/qwen35/decoder.hpp:78-84); NULL updates in place.
 * q, k: [key_heads][head_dim], already normalised; v, y: [value_heads]
 * [head_dim]; decay, beta: [value_heads]. Value head h reads key head
 * h % key_heads (src/models/qwen35/decoder.cpp:221). All device pointers. */
typedef struct gufo_cuda_delta_seq {
  float* state;
  float* state_out;
  const float* q;
  const float* k;
  const float* v;
  const float* decay;
  const float* beta;
  float* y;
} gufo_cuda_delta_seq;

/* Applies the delta rule to `nseq` independent sequences in one launch.
 * `seqs` is a host array of `nseq` descriptors (device pointers inside). */
int gufo_cuda_delta_rule_device(gufo_cuda_ctx* ctx,
                                const gufo_cuda_delta_seq* seqs, int nseq,
                                int key_heads, int value_heads, int head_dim);

/* The small weights Mixer loads per DeltaNet layer
 * (src/models/qwen35/decoder.cpp:40-47,76-80): host pointers, copied. */
typedef struct gufo_cuda_deltanet_params {
  int key_heads;
  int value_heads;
  int head_dim;
  int conv_kernel;
  float rms_eps;
  const float* conv;     /* [2 key_dim + value_dim][conv_kernel] */
  const float* ssm_a;    /* [value_heads] */
  const float* dt_bias;  /* [value_heads] */
  const float* ssm_norm; /* [head_dim] */
} gufo_cuda_deltanet_params;

int gufo_cuda_deltanet_layer_create(gufo_cuda_ctx* ctx,
                                    const gufo_cuda_deltanet_params* params,
                                    gufo_cuda_deltanet_layer* out);
int gufo_cuda_deltanet_layer_free(gufo_cuda_ctx* ctx,
                                  gufo_cuda_deltanet_layer layer);

/* One sequence's step through Mixer::Linear
 * (src/models/qwen35/decoder.cpp:161-265): causal conv + SiLU, q/k L2 norm,
 * gates, delta rule, gated RMSNorm. `in` is the kLinearIn row
 * [qkv | z | alpha | beta]; y gets value_dim values. The conv window is read
 * from conv_in and the advanced window written to conv_out, two distinct
 * [conv_kernel - 1][channels] buffers (the reference's fused step also writes
 * a second window and swaps, src/models/qwen35_2b/deltanet.cpp:236-247,355);
 * keeping conv_in is the rollback of a draft token. ssm / ssm_out as `state` /
 * `state_out` above. All device pointers. */
typedef struct gufo_cuda_linear_seq {
  const float* in;
  const float* conv_in;
  float* conv_out;
  float* ssm;
  float* ssm_out;
  float* y;
} gufo_cuda_linear_seq;

int gufo_cuda_deltanet_linear_device(gufo_cuda_ctx* ctx,
                                     gufo_cuda_deltanet_layer layer,
                                     const gufo_cuda_linear_seq* seqs,
                                     int nseq);

/* DeltaNetStep::Run (src/models/qwen35_2b/deltanet.hpp:42-44,
 * deltanet.cpp:358-392): 1 to 4 tokens of a sequence through the layer, the
 * gates taken from the residual stream. Per token t: normed = RMSNorm(h[t]) *
 * attn_norm, alpha / beta = the F32 ssm_alpha / ssm_beta rows times normed,
 * then Mixer::Linear on in[t] (only its [qkv | z] part is read). Tokens before
 * the last advance ssm in place. With two or more tokens the last one is a
 * draft: ssm keeps the state before it and ssm_spec gets the state after it,
 * conv_saved the window before it and conv_out the window after it (the
 * reference's two-token form; accepting the draft is ssm <- ssm_spec, rejecting
 * it conv <- conv_saved). With one token: ssm in place, conv_in -> conv_out,
 * conv_saved / ssm_spec unused (may be NULL). conv_in, conv_out and conv_saved
 * are distinct buffers. One launch per token index over all sequences. */
typedef struct gufo_cuda_deltanet_step_seq {
  int n_tokens;          /* 1 .. 4 */
  const float* in;       /* [n_tokens] rows, in_stride floats apart */
  int64_t in_stride;
  const float* h;        /* [n_tokens] residual rows, h_stride floats apart */
  int64_t h_stride;
  const float* conv_in;
  float* conv_out;
  float* conv_saved;
  float* ssm;
  float* ssm_spec;
  float* y;              /* [n_tokens] rows of value_dim values, y_stride apart */
  int64_t y_stride;
} gufo_cuda_deltanet_step_seq;

int gufo_cuda_deltanet_step_device(gufo_cuda_ctx* ctx,
                                   gufo_cuda_deltanet_layer layer,
                                   gufo_cuda_matrix ssm_alpha,
                                   gufo_cuda_matrix ssm_beta,
                                   const float* attn_norm, float rms_eps,
                                   const gufo_cuda_deltanet_step_seq* seqs,
                                   int nseq);

/* ---- the small steps between the products ------------------------------- */

/* The CPU work Decoder::Step does between its Projections calls, as device
 * operations on the context's stream, so that a host-side decode loop (for
 * example one that all-gathers row-split products between them) never leaves
 * the device. All pointers are device pointers. */

/* h = row *device_token of `matrix`, dequantized (the embedding lookup,
 * src/models/qwen35/decoder.cpp:486-489). */
int gufo_cuda_embed_device(gufo_cuda_ctx* ctx, gufo_cuda_matrix matrix,
                           const int* device_token, float* h);
/* h += delta (delta may be NULL), then normed = RMS(h) * weight (vec::RmsNorm,
 * src/core/vec.hpp:57-63, with the residual add of decoder.cpp:504-506).
 * `advance` (may be NULL) is an int counter incremented afterwards. */
int gufo_cuda_add_rms_norm_device(gufo_cuda_ctx* ctx, float* h,
                                  const float* delta, const float* weight,
                                  float eps, int n, float* normed, int* advance);
/* act[i] = silu(ffn[i]) * ffn[f + i] (decoder.cpp:511-514). */
int gufo_cuda_swiglu_device(gufo_cuda_ctx* ctx, const float* ffn, int f,
                            float* act);

/* Mixer::Attention for one token (src/models/qwen35/decoder.cpp:267-412): q/k
 * RMSNorm and RoPE, the fp16 cache append at *position, softmax over positions
 * 0..*position in slices, the output gate. `in` is the kAttentionIn row
 * [q and gate | k | v]; `ctx_out` gets heads * head_dim values. */
typedef struct gufo_cuda_attention_args {
  int heads, kv_heads, head_dim, rope_dim, max_positions;
  float rms_eps;
  const int* position;   /* device int: rows already in the cache */
  const float* in;
  const float* q_norm;   /* [head_dim] */
  const float* k_norm;   /* [head_dim] */
  const float* inv_freq; /* [rope_dim / 2]: 1 / theta^(2i / rope_dim) */
  void* keys;            /* fp16 [max_positions][kv_heads * head_dim] */
  void* values;
  float* queries;        /* scratch [heads][head_dim] */
  float* partials;       /* scratch [kv_heads][32][heads / kv_heads][head_dim + 2] */
  float* ctx_out;
} gufo_cuda_attention_args;

int gufo_cuda_attention_device(gufo_cuda_ctx* ctx,
                               const gufo_cuda_attention_args* args);

/* ---- routed experts (MoE models) ---------------------------------------- */

/* Route and SharedExpertScale (src/models/qwen35/moe.cpp:16-47) for `tokens`
 * rows of router outputs on the device, `stride` floats apart: softmax in
 * double over the first `experts` values of a row, the `k` most probable
 * experts in descending order (ties: lower id), their weights renormalised
 * with the sum floored at 6.103515625e-5 (experts <= 1024). chosen and weights
 * are [tokens][k] on the device. shared_scale (may be NULL) gets, per token, the
 * sigmoid of the row's value at index `experts` (the shared expert's gate,
 * Stage::kRouter's last output). */
int gufo_cuda_route_device(gufo_cuda_ctx* ctx, const float* router, int stride,
                           int tokens, int experts, int k, int* chosen,
                           float* weights, float* shared_scale);

/* The stacked expert tensors of one layer, each [cols, rows, experts] in GGUF
 * terms and uploaded as one matrix of rows * experts rows
 * (src/models/qwen35/gguf_projections.cpp:132-139,229-233). */
typedef struct gufo_cuda_expert_bank {
  gufo_cuda_matrix gate_exps;  /* [hidden, expert_ffn, experts] */
  gufo_cuda_matrix up_exps;    /* [hidden, expert_ffn, experts] */
  gufo_cuda_matrix down_exps;  /* [expert_ffn, hidden, experts] */
  int experts;
  int expert_ffn;
  int hidden;
} gufo_cuda_expert_bank;

/* The loop body of Decoder::MoeFfn (src/models/qwen35/decoder.cpp:545-551,
 * i.e. ApplyExpert(kExpertIn), SwiGLU, ApplyExpert(kExpertDown)) for `pairs`
 * (input row, expert) pairs in two grouped launches: y[p] = down_e(silu(gate_e
 * x_p) * up_e x_p) with e = ids[p], read from DEVICE memory at run time, so
 * the ids may come straight from gufo_cuda_route_device. ids[p] < 0 skips the
 * pair and leaves y[p] untouched (expert-parallel ranks pass -1 for experts
 * they do not hold). x_p = x + (p / pairs_per_input) * x_stride: a batch of
 * tokens with k slots each passes x_stride = hidden and pairs_per_input = k;
 * x_stride 0 shares one input. Scratch: ffn [pairs][2 * expert_ffn], act
 * [pairs][expert_ffn]; which of the two holds intermediate values afterwards
 * depends on the kernels taken (Q4_K banks activate inside the gate / up
 * launch and leave ffn untouched). */
int gufo_cuda_expert_ffn_device(gufo_cuda_ctx* ctx,
                                const gufo_cuda_expert_bank* bank,
                                const int* ids, int pairs, const float* x,
                                int64_t x_stride, int pairs_per_input,
                                float* ffn, float* act, float* y);

/* Decoder::MoeFfn behind the router (decoder.cpp:535-557) in one call: out[t] =
 * shared[t] * scale[t] + sum over slots s, in slot order, of weights[t][s] *
 * y(t, s), y(t, s) the FFN of expert ids[t][s] applied to x_t = x + t *
 * x_stride; a slot with ids < 0 adds nothing. Equal to
 * gufo_cuda_expert_ffn_device (pairs = tokens * k, pairs_per_input = k) followed
 * by gufo_cuda_moe_combine_device up to the rounding of the row sums' order;
 * for Q4_K banks with expert_ffn 256 or 512 and k <= 8 it runs as two launches
 * (gate / up with the SwiGLU; the down rows of a token's experts with the
 * weighted sum) and touches neither ffn nor expert_out. Scratch as for
 * gufo_cuda_expert_ffn_device plus expert_out [tokens][k][hidden]. out may be
 * shared. */
int gufo_cuda_moe_ffn_device(gufo_cuda_ctx* ctx,
                             const gufo_cuda_expert_bank* bank, const int* ids,
                             const float* weights, const float* scale,
                             int tokens, int k, const float* x, int64_t x_stride,
                             const float* shared, float* ffn, float* act,
                             float* expert_out, float* out);

/* out[t] = shared[t] * scale[t] + sum over slots, in slot order, of
 * weights[t][slot] * expert_out[t][slot] (decoder.cpp:541-556). out may be
 * shared. */
int gufo_cuda_moe_combine_device(gufo_cuda_ctx* ctx, const float* shared,
                                 const float* scale, const float* weights,
                                 const float* expert_out, int tokens, int k,
                                 int hidden, float* out);

/* ---- row-split ranks: all-gather over NVLink peer memory ------------------- */

/* For hosts that split a stage's rows over several GPUs (one process per GPU)
 * and need every rank to see the whole output vector: each rank stores its
 * slice straight into every rank's copy of the vector over NVLink and raises a
 * flag there, one small kernel per gather on the context's stream (it can be
 * captured in a CUDA graph). The reference has no counterpart (it runs on one
 * accelerator); the products it follows are Projections::Apply's.
 *
 * Every rank allocates an arena of the same size with gufo_cuda_malloc, exports
 * it (gufo_cuda_ipc_export), exchanges the 64-byte handles by its own means, and
 * creates the group from all ranks' handles in rank order (its own entry is
 * ignored). The first GUFO_CUDA_PEER_HEADER_BYTES of an arena belong to the
 * group; full vectors live behind them at the same offset on every rank. All
 * ranks must have created their group (which clears the whole arena) before any
 * of them gathers: put a barrier of the host's own between the two. A flag that
 * does not arrive within the limit (about four seconds unless
 * gufo_cuda_peer_group_set_limit changed it) ends the wait:
 * gufo_cuda_peer_group_status then returns GUFO_CUDA_TIMEOUT, and every later
 * gather gives up at once, its output invalid, until every rank has called
 * gufo_cuda_peer_group_reset (all ranks together, none of them gathering: it
 * clears the flags, the gather count and the error word of the rank's arena).
 *
 * gufo_cuda_peer_group_create_local builds the same group from device pointers
 * the process can already reach (`arenas[r]` for every rank r, its own
 * included): for one process that drives several GPUs with peer access enabled,
 * and for tests. */
#define GUFO_CUDA_IPC_HANDLE_BYTES 64
#define GUFO_CUDA_PEER_HEADER_BYTES 4096
typedef struct gufo_cuda_peer_group gufo_cuda_peer_group;
int gufo_cuda_ipc_export(gufo_cuda_ctx* ctx, const void* device_ptr, void* handle);
int gufo_cuda_peer_group_create(gufo_cuda_ctx* ctx, int rank, int world,
                                void* own_arena, size_t arena_bytes,
                                const void* handles, gufo_cuda_peer_group** out);
int gufo_cuda_peer_group_create_local(gufo_cuda_ctx* ctx, int rank, int world,
                                      void* const* arenas, size_t arena_bytes,
                                      gufo_cuda_peer_group** out);
int gufo_cuda_peer_group_destroy(gufo_cuda_peer_group* group);
/* How long a gather waits for a peer's flag, in microseconds of SM clocks. */
int gufo_cuda_peer_group_set_limit(gufo_cuda_peer_group* group, int64_t microseconds);
int gufo_cuda_peer_group_reset(gufo_cuda_peer_group* group);
/* Rank r's `slice_floats` values at local_src land at arena_offset (bytes) +
 * r * slice_floats * 4 in every rank's arena; returns once enqueued. The kernel
 * ends when the slices of all ranks have arrived in this rank's arena. */
int gufo_cuda_peer_allgather_device(gufo_cuda_peer_group* group,
                                    const float* local_src, size_t arena_offset,
                                    size_t slice_floats);
int gufo_cuda_peer_group_status(gufo_cuda_peer_group* group);
/* The product and the gather in one kernel: a one-token product with a fused
 * input (gufo_cuda_matmul_fused_device; up to four Q4_K or Q6_K parts of one
 * block format) whose thread blocks store this rank's rows straight into every
 * rank's copy of the full vector (arena_offset bytes into each arena, rank r's
 * rows at r * rows * 4 behind it: plain peer stores over NVLink) and whose last
 * thread block raises this rank's flag of `slot` (0..7, one per vector that can
 * be in flight) in every arena. No rank waits inside this kernel. A kernel that
 * reads the full vector must first wait for the slot: pass `wait_slot` to the
 * next gufo_cuda_matmul_gather_device whose input it is (the wait then sits in
 * that kernel's prologue), or enqueue gufo_cuda_peer_wait_device (a one-block
 * kernel that waits) ahead of other readers. wait_slot < 0: the input is local.
 * A slot's vector may be rewritten once every rank has launched a later gather
 * of another slot (a rank raises a flag only after all its earlier kernels,
 * readers included, have finished). Waits are bounded and report through
 * gufo_cuda_peer_group_status as above. The reference has no counterpart. */
int gufo_cuda_matmul_gather_device(gufo_cuda_peer_group* group, const gufo_cuda_rows* parts,
                                   int nparts, const gufo_cuda_fused_input* input,
                                   size_t arena_offset, int slot, int wait_slot);
int gufo_cuda_peer_wait_device(gufo_cuda_peer_group* group, int slot);
/* The same one-token fused product with its rows kept local (device_y, this
 * rank's memory) and the bounded wait for `wait_slot` in its prologue: the
 * consumer of vectors that the ranks' earlier products stored into the arenas.
 * With ranks that split the heads of a layer and the columns of its output and
 * down projections, every rank's gufo_cuda_matmul_gather_device product stores
 * its partial sums (all rows, its share of the columns) as rank r's run of a
 * [world][rows] vector, and the next product adds them to the residual in rank
 * order (gufo_cuda_fused_input.delta_parts = world, delta_stride = rows): two
 * exchanges per layer instead of four gathers, and no rank multiplies another
 * rank's heads. The reference has no counterpart. */
int gufo_cuda_matmul_wait_device(gufo_cuda_peer_group* group, const gufo_cuda_rows* parts,
                                 int nparts, const gufo_cuda_fused_input* input,
                                 int wait_slot, float* device_y);

/* ---- device-resident decode step ---------------------------------------- */

/* Shape of a Qwen3.5-family model: the fields of qwen35::Config
 * (src/models/qwen35/config.hpp:13-62) the decode step reads, plus the capacity
 * of the attention cache. */
typedef struct gufo_cuda_decoder_config {
  int layers;
  int hidden;
  int ffn;
  int vocab;
  float rms_eps;
  int full_attention_interval;
  int heads;
  int kv_heads;
  int head_dim;
  int rope_dim;
  float rope_theta;
  int conv_kernel;
  int linear_key_heads;
  int linear_value_heads;
  int linear_head_dim;
  int max_positions; /* attention cache rows per layer */
  int use_graph;     /* replay the step as a CUDA graph after the first steps */
  /* MoE models (qwen35moe): 0 experts for a dense model. `ffn` is then the
   * shared expert's width (Config::FfnWidth, config.hpp). */
  int experts;
  int experts_used;
  int expert_ffn;
} gufo_cuda_decoder_config;

/* One layer's weights: matrix handles of this context (0 where the layer kind
 * has none) and host fp32 vectors, copied. Names are the GGUF tensor names the
 * reference loads (src/models/qwen35/gguf_projections.cpp:100-175,
 * decoder.cpp:67-98,441-455). */
typedef struct gufo_cuda_layer_weights {
  gufo_cuda_matrix attn_qkv, attn_gate, ssm_alpha, ssm_beta, ssm_out; /* DeltaNet */
  gufo_cuda_matrix attn_q, attn_k, attn_v, attn_output;               /* attention */
  gufo_cuda_matrix ffn_gate, ffn_up, ffn_down; /* dense FFN, or the shared expert */
  /* MoE layers: the router [hidden, experts] and the shared expert's gate
   * [hidden, 1] (both F32), and the stacked expert tensors. */
  gufo_cuda_matrix ffn_gate_inp, ffn_gate_inp_shexp;
  gufo_cuda_matrix ffn_gate_exps, ffn_up_exps, ffn_down_exps;
  const float* attn_norm;           /* [hidden] */
  const float* post_attention_norm; /* [hidden] */
  const float* ssm_conv1d;          /* [channels][conv_kernel] */
  const float* ssm_a;               /* [value heads] */
  const float* ssm_dt_bias;         /* [value heads] */
  const float* ssm_norm;            /* [head dim] */
  const float* attn_q_norm;         /* [head_dim] */
  const float* attn_k_norm;         /* [head_dim] */
} gufo_cuda_layer_weights;

typedef struct gufo_cuda_decoder_weights {
  gufo_cuda_matrix token_embd;
  gufo_cuda_matrix output;      /* 0 when the LM head is token_embd */
  const float* output_norm;     /* [hidden] */
  const gufo_cuda_layer_weights* layers; /* [config.layers] */
} gufo_cuda_decoder_weights;

typedef struct gufo_cuda_decoder gufo_cuda_decoder;

/* qwen35::Decoder (src/models/qwen35/decoder.hpp:105-132) with every buffer on
 * the device: the residual stream, the DeltaNet states and conv windows, the
 * fp16 attention cache and the logits stay in HBM between steps, as the
 * reference's NPU decoders keep the residual stream on their device
 * (src/models/qwen35_2b/npu_decoder.hpp:18-21). Dense and MoE models; in a
 * MoE layer the router, the top-k and the routed experts run on the device
 * too (Decoder::MoeFfn, decoder.cpp:535-557). The matrices must outlive the
 * decoder. Holds one sequence (DecodeState). */
int gufo_cuda_decoder_create(gufo_cuda_ctx* ctx,
                             const gufo_cuda_decoder_config* config,
                             const gufo_cuda_decoder_weights* weights,
                             gufo_cuda_decoder** out);
int gufo_cuda_decoder_destroy(gufo_cuda_decoder* decoder);
/* A fresh sequence: Mixer::NewState (src/models/qwen35/decoder.cpp:144-159). */
int gufo_cuda_decoder_reset(gufo_cuda_decoder* decoder);
/* Decoder::Step (src/models/qwen35/decoder.cpp:478-528): runs `token` at the
 * current position, advances the state, and leaves the vocab logits in
 * host_logits (may be NULL to leave them on the device only). Pageable memory
 * gets a copy after the step. Pinned memory that the device can address
 * (cudaHostAlloc, cudaHostRegister; 16-byte aligned) is written by the LM
 * head's own stores while that kernel runs, once the step replays as a graph:
 * pass the same buffer step after step (a new buffer costs a graph capture).
 * Returns GUFO_CUDA_BAD_ARGUMENT for a token outside [0, vocab) and
 * GUFO_CUDA_TOO_LARGE when the attention cache is full. */
int gufo_cuda_decoder_step(gufo_cuda_decoder* decoder, int token,
                           float* host_logits);
/* NpuDecoder::Step(tokens, count, state, logits)
 * (src/models/qwen35_2b/npu_decoder.hpp:57-65, npu_decoder.cpp:558-628): runs
 * `count` (1 or 2) tokens from the current position in one pass, every weight
 * read once for both; token t's logits land at t * vocab (host_logits may be
 * NULL to leave them on the device). With want_logits == 0 the LM head is
 * skipped (prompt passes) and host_logits must be NULL; the final residuals
 * are kept either way (gufo_cuda_decoder_hidden_device). With two tokens the
 * second stays a draft until gufo_cuda_decoder_resolve, which must come
 * before the next step. Errors as gufo_cuda_decoder_step. */
int gufo_cuda_decoder_step_tokens(gufo_cuda_decoder* decoder, const int* tokens,
                                  int count, int want_logits,
                                  float* host_logits);
/* With the context option "step_kernel" = 1, one-token steps of a dense model
 * whose stages hold one block format each (Q4_K or Q6_K; F32 alpha / beta rows)
 * run as ONE persistent kernel, launched cooperatively with one thread block
 * per SM, instead of a chain of launches: the reference's own NPU decoder
 * submits a layer at a time for the same reason
 * (src/models/qwen35_2b/npu_decoder.hpp:18-25). Other models and two-token
 * steps take the launch chain regardless. The option is off unless set: on
 * B200 a grid-wide barrier costs what a programmatic kernel boundary does and
 * the chain is the faster of the two. Every wait inside the kernel is bounded (option "step_wait_us",
 * two seconds unless set): a wait that runs out ends the kernel, and the step
 * call that downloads the logits, or gufo_cuda_decoder_status, returns
 * GUFO_CUDA_TIMEOUT once; the outputs and states of that step are invalid
 * (gufo_cuda_decoder_reset starts over), the decoder and the context stay
 * usable. gufo_cuda_decoder_status waits for the stream and reports such a
 * failure of steps that left their logits on the device. */
int gufo_cuda_decoder_status(gufo_cuda_decoder* decoder);
/* The operations of the last step run by the persistent kernel, in order: the
 * stage each belongs to (a GUFO_CUDA_TIMELINE_* kind, as
 * gufo_cuda_decoder_timeline reports for the launch chain; the reference keeps
 * the same split, NpuDecoder::Timeline, npu_decoder.hpp:121-154), the weight or
 * state bytes it moves, and its device time in microseconds from block 0's
 * clock stamps, barrier to barrier. Up to `capacity` entries are written
 * (arrays may be NULL); *count receives the number of operations, 0 when the
 * model runs on the launch chain. */
int gufo_cuda_decoder_step_profile(gufo_cuda_decoder* decoder, int capacity,
                                   int* stages, int64_t* bytes, double* us,
                                   int* count);
/* NpuDecoder::Resolve (npu_decoder.cpp:630-650) after a two-token step:
 * keep_second != 0 keeps the draft (the DeltaNet draft states become the
 * states), 0 rolls the decoder back to just after the first token (its conv
 * windows, one position less; the draft's attention cache rows are overwritten
 * by the next step). */
int gufo_cuda_decoder_resolve(gufo_cuda_decoder* decoder, int keep_second);
/* NpuDecoder::hidden(t) (npu_decoder.hpp:70-72): device address of the final
 * residual (before output_norm, `hidden` fp32) of token t of the last step:
 * the MTP head's input. Valid until the next step. */
int gufo_cuda_decoder_hidden_device(gufo_cuda_decoder* decoder, int t,
                                    const float** hidden);
/* Device address of the last step's logits (vocab fp32 per token). */
int gufo_cuda_decoder_logits_device(gufo_cuda_decoder* decoder,
                                    const float** device_logits);
int gufo_cuda_decoder_position(const gufo_cuda_decoder* decoder);
/* Device time per stage of the step, by CUDA events between the stages: the
 * split the reference's NpuDecoder::Timeline keeps
 * (src/models/qwen35_2b/npu_decoder.hpp:121-154). While enabled, steps are
 * launched eagerly (no graph replay). The call returns the totals in
 * milliseconds and the number of steps accumulated so far (either pointer may
 * be NULL), then switches collection on or off; switching clears the totals. */
enum {
  GUFO_CUDA_TIMELINE_EMBED = 0,
  GUFO_CUDA_TIMELINE_IN = 1,        /* norm + kLinearIn / kAttentionIn */
  GUFO_CUDA_TIMELINE_DELTANET = 2,
  GUFO_CUDA_TIMELINE_ATTENTION = 3,
  GUFO_CUDA_TIMELINE_OUT = 4,       /* kMixerOut */
  GUFO_CUDA_TIMELINE_FFN_IN = 5,    /* residual + norm + kFfnIn */
  GUFO_CUDA_TIMELINE_FFN_DOWN = 6,  /* SwiGLU + kFfnDown */
  GUFO_CUDA_TIMELINE_LM_HEAD = 7,   /* residual + norm + kLmHead */
  GUFO_CUDA_TIMELINE_KINDS = 8
};
int gufo_cuda_decoder_timeline(gufo_cuda_decoder* decoder, int enable,
                               double* stage_ms, int* steps);
/* Copies DeltaNet layer `layer`'s conv window [conv_kernel - 1][channels] and
 * state [value heads][dk][dk] to the host (either may be NULL): the checkpoint
 * read of src/models/qwen35/state_capture.hpp:8-14. */
int gufo_cuda_decoder_linear_state(gufo_cuda_decoder* decoder, int layer,
                                   float* host_conv, float* host_ssm);

#ifdef __cplusplus
}
#endif
#endif /* GUFO_CUDA_H_ */
