#pragma once

#include <vector>

#include "core/gguf.hpp"
#include "cuda/cuda_projections.hpp"

struct gufo_cuda_decoder;

// qwen35::Decoder (src/models/qwen35/decoder.hpp:105-132) with the whole step on
// a B200: residual stream, DeltaNet states, conv windows, the fp16 attention
// cache and the logits stay in device memory between steps, as the NPU decoders
// keep theirs on the accelerator (src/models/qwen35_2b/npu_decoder.hpp:18-21).
// Dense and MoE models. The decoder holds one sequence; Reset starts a new one.
// The matrices are the ones `projections` uploaded, so it must outlive the
// decoder; the GGUF file is only read during construction.
namespace gufo_npu::cuda {

class Decoder {
public:
  Decoder(const gguf::File& file, const CudaProjections& projections,
          int max_positions = 4096);
  ~Decoder();
  Decoder(const Decoder&) = delete;
  Decoder& operator=(const Decoder&) = delete;

  // Runs `token` at the current position and returns the vocab logits
  // (Decoder::Step). Throws std::out_of_range for a token outside the
  // vocabulary, std::length_error when the attention cache is full.
  const std::vector<float>& Step(int token);
  // `count` (1 or 2) tokens from the current position in one pass, the weights
  // read once for both (NpuDecoder::Step, src/models/qwen35_2b/
  // npu_decoder.hpp:57-65). Returns token t's logits at t * vocab, or nullptr
  // without `logits` (prompt passes; the LM head is skipped). After two tokens
  // the second is a draft until Resolve. Throws std::invalid_argument for
  // another count.
  const float* Step(const int* tokens, int count, bool logits = true);
  // After a two-token Step: keep the second token, or roll the decoder back to
  // just after the first (NpuDecoder::Resolve, npu_decoder.hpp:66-68).
  void Resolve(bool keep_second);
  // The final residual (before output_norm) of token t of the last Step, copied
  // to the host: the MTP head's input (NpuDecoder::hidden, npu_decoder.hpp:70-72).
  const std::vector<float>& hidden(int t = 0);
  // A fresh sequence (Mixer::NewState).
  void Reset();
  int position() const;

private:
  const CudaProjections& projections_;
  gufo_cuda_decoder* decoder_ = nullptr;
  std::vector<float> logits_;
  std::vector<float> pair_logits_;
  std::vector<float> hidden_;
  int hidden_width_ = 0;
};

}  // namespace gufo_npu::cuda
