// Launch interface of the GEMV kernels, shared by the C-ABI entry points and
// the device-resident decoder.
#pragma once

#include "common.cuh"

namespace gufo {

constexpr int kMaxParts = 8;
constexpr int kMaxTokens = 8;

struct GemvPart {
  const uint8_t* data;  // first row of the range
  int rows;
  int out_offset;       // column of y where this part starts
  int type;
  int row_bytes;
};

struct GemvArgs {
  GemvPart parts[kMaxParts];
  int nparts;
  int total_rows;   // sum of these parts' rows
  int y_stride;     // width of a y row
  int cols;
  const float* x;   // [tokens][cols]
  float* y;         // [tokens][total_rows]
  // Grouped products (see FastGemvArgs): null for an ordinary product.
  const int* group_ids = nullptr;
  int groups = 0;
  int x_group_stride = 0;
  int x_group_div = 1;
  int y_group_stride = 0;
};

// Enqueues, for every group g with group_ids[g] >= 0 (device memory), the
// one-token product of matrix group_ids[g] of each stacked part with the group's
// input; `prologue` is kProloguePlain (x fp32) or kPrologueSwiGlu (x = [gate |
// up] per group; `scratch` then holds groups * cols activated values for parts
// the tensor-core kernel does not run). Fill the group fields of `args`.
int LaunchGemvGrouped(gufo_cuda_ctx* ctx, const GemvArgs& args, int prologue, float* scratch,
                      bool activate = false);
// Whether that product can store silu(gate) * up of its two parts by itself
// (`activate`: y then holds rows / 2 values per group).
bool GroupedSwiGluInProduct(const gufo_cuda_ctx* ctx, const GemvArgs& args);

// Enqueues y = [W_0 x | W_1 x | ...] for `tokens` rows; x and y on the device.
// The caller holds ctx->mu.
int LaunchGemv(gufo_cuda_ctx* ctx, const GemvArgs& base, int tokens);

int StageActivations(gufo_cuda_ctx* ctx, const float* x, int tokens, int cols,
                     int group, float extra, const uint8_t** image);

// Fills `args` (parts, widths) from matrix handles; ctx->mu is held.
int BuildGemvArgs(gufo_cuda_ctx* ctx, const gufo_cuda_rows* parts, int nparts,
                  GemvArgs* args);

}  // namespace gufo
