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
  // A fresh sequence (Mixer::NewState).
  void Reset();
  int position() const;

private:
  const CudaProjections& projections_;
  gufo_cuda_decoder* decoder_ = nullptr;
  std::vector<float> logits_;
};

}  // namespace gufo_npu::cuda
