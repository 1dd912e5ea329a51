// Interface of the persistent decode-step kernel (step_kernel.cu): a whole
// Decoder::Step (src/models/qwen35/decoder.cpp:478-528 in the reference) as one
// cooperative launch. The host describes the step as a program of operations
// in device memory; every thread block walks the program, with a grid-wide
// barrier where kernel boundaries used to be, and streams the weights of later
// operations into its shared-memory ring while it waits.
#pragma once

#include "decode_device.cuh"
#include "mma_common.cuh"

namespace gufo {

constexpr int kStepTeams = 2;                         // teams of eight warps per block
constexpr int kStepConsumerWarps = kStepTeams * kTeamWarps;
constexpr int kStepReducerWarp = kStepConsumerWarps;  // sums the teams' partial rows, writes y
constexpr int kStepProducerWarp = kStepConsumerWarps + 1;   // issues every bulk copy
constexpr int kStepThreads = (kStepConsumerWarps + 2) * 32;
constexpr int kStepSlots = 3;                         // ring slots per team
constexpr int kStepExchange = 4;                      // partial-row buffers per team
constexpr int kStepSlotBytes = 16 * (kQ6KSlabBlocks * kQ6KBytes + 16);   // the larger (Q6_K) slab
constexpr int kStepMaxTokens = 1;

enum StepOpKind {
  kStepEmbed = 0,      // arg: unused (the program's embed)
  kStepGemv = 1,       // arg: index into gemv
  kStepDelta = 2,      // arg: index into delta
  kStepAttnPrep = 3,   // arg: index into attn
  kStepAttnSlice = 4,
  kStepAttnMerge = 5,
};

// Prologues of a product beyond FastPrologue (common.cuh): the gated RMSNorm
// over each DeltaNet head's outputs, x = RMS_head(y) * w * silu(z)
// (src/models/qwen35/decoder.cpp:258-263), applied while the output
// projection's input is staged.
constexpr int kPrologueGatedNorm = 4;

struct StepGemv {
  FastPart parts[kFastMaxParts];
  int nparts;
  int type;              // GUFO_CUDA_Q4_K or GUFO_CUDA_Q6_K (every part)
  int cols;
  int row_bytes;
  int tiles;             // 16-row tiles over all parts
  int slabs_per_tile;    // slabs of up to eight 256-value blocks
  // split != 0: every (tile, slab) is an item of its own; slab s writes its
  // partial rows to y + s * y_split_stride, and the consumer adds the parts.
  int split;
  float* y;
  int y_stride;          // floats between tokens
  int y_split_stride;
  int prologue;          // FastPrologue or kPrologueGatedNorm
  const float* x;        // plain / SwiGLU / gated norm input
  const float* h_in;     // kPrologueResNorm: residual ...
  const float* delta;    //   ... plus delta_parts vectors delta_stride floats apart (may be null)
  int delta_parts;
  int delta_stride;
  const float* norm_w;
  float eps;
  float* h_out;          // written by block 0
  float* normed_out;     // written by block 0 (may be null)
  int* advance;          // incremented by block 0 (may be null)
  const float* z;        // kPrologueGatedNorm: the gate rows (z_stride floats between tokens),
  const float* gate_w;   //   the norm weights [head_dim]
  int gate_head_dim;
  int z_stride;
};

struct StepDelta {
  const float* in;        // the input product's row [q | k | v | z]
  const float* gate_x;    // the layer's normed input [cols]
  const float* alpha_w;   // [value heads][cols] F32
  const float* beta_w;
  int cols;
  const float* conv_w;    // [channels][kernel]
  const float* ssm_a;
  const float* dt_bias;
  float* conv[2];         // the two windows: conv[parity] is read, conv[parity ^ 1] written
  float* state;           // [value heads][dk][dk]
  float* y;               // [value heads][dk], before the gated norm
  int key_heads, value_heads, head_dim, conv_kernel;
};

struct StepOp {
  int kind;
  int items;   // independent pieces of work, dealt round-robin to the grid's teams
  int rot;     // item i belongs to team (i + rot) % teams, numbered 2 * block + team
  int arg;
};

struct StepProgram {
  const StepOp* ops;
  int nops;
  const StepGemv* gemv;
  const StepDelta* delta;
  const AttnArgs* attn;
  EmbedArgs embed;
  // sync[0]: arrivals at the grid barriers; sync[1]: blocks that have left;
  // sync[2]: error word (0, or the code of the first wait that ran out).
  unsigned* sync;
  unsigned long long* stamps;   // [nops + 1] nanosecond stamps of block 0 (may be null)
  int parity;                   // which conv window is current
  int region_bytes;             // shared memory for the staged input / team scratch
  long long wait_limit;         // clock cycles any wait may take
  int skip_arrival_at;          // test hook: block 0 stays away from this barrier (-1: off)
};

// Codes left in the error word.
constexpr unsigned kStepErrGridBarrier = 1;
constexpr unsigned kStepErrSlotFull = 2;
constexpr unsigned kStepErrSlotEmpty = 3;
constexpr unsigned kStepErrExchange = 4;
constexpr unsigned kStepErrReducer = 5;

// Shared memory of one launch with `region_bytes` for the staged input.
size_t StepSharedBytes(int region_bytes);
// Bytes a product's staged input needs in the region (image + the Q6_K plane of zeros).
int StepImageBytes(int type, int cols);
// Bytes the teams' scratch needs in the region.
int StepScratchBytes();
// Thread blocks of the launch on `device` (one per SM), 0 when the kernel cannot run there.
int StepGridBlocks(int device, int region_bytes);
// Enqueues the step; the caller holds ctx->mu. Cooperative launch.
int LaunchStep(gufo_cuda_ctx* ctx, const StepProgram& program, int grid);

}  // namespace gufo
