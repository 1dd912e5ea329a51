// Launch interface of the tcgen05 small-M GEMM (16 to 128 token rows per
// weight read).
#pragma once

#include "gemv.cuh"
#include "mma_common.cuh"

namespace gufo {

// Fewest token rows that take this path; below, the GEMV kernels re-read the
// weights once per 8 tokens and are faster. Measured: 2 x 9728 x 2560 Q4_K costs
// 27 us per 8-token pass against 31 us here whatever the rows (so from a second
// pass on this path wins, and the third is where it is taken); 248320 x 2560
// Q6_K 330 us per pass against 670 us here (from a third pass on).
constexpr int kTcMinTokens = 17;       // Q4_K parts
constexpr int kTcMinTokensQ6K = 17;    // Q6_K parts
constexpr int kTcMaxTokens = 128;   // token rows per pass (the MMA's N)

// Whether a product of `tokens` rows against parts of `type` runs on this path.
bool TcGemmRuns(const gufo_cuda_ctx* ctx, int type, int cols, int tokens);

// Enqueues y = [W_0 x | W_1 x | ...] for `tokens` >= kTcMinTokens rows; every
// part of `base` must satisfy TcGemmRuns. x is 16-byte aligned.
int LaunchGemmTc(gufo_cuda_ctx* ctx, const GemvArgs& base, int tokens);

// Reads (after synchronizing the stream) the code a bounded wait of the GEMM
// kernel left when it ran out; 0 when none did.
int TcGemmError(gufo_cuda_ctx* ctx, int* code);

}  // namespace gufo
