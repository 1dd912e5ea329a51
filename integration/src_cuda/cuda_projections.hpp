#pragma once

#include <memory>
#include <vector>

#include "core/gguf.hpp"
#include "models/qwen35/config.hpp"
#include "models/qwen35/projections.hpp"

struct gufo_cuda_ctx;

// A Qwen3.5 / Qwen3.6 model's matrix products on a B200 through libgufo_cuda
// (include/gufo_cuda.h): the CUDA counterpart of GgufProjections
// (src/models/qwen35/gguf_projections.hpp). Construction checks every
// projection tensor's shape like GgufProjections and uploads the tensors once
// (Q4_K, Q6_K, Q5_K, Q8_0 and F32 rows; other types throw std::runtime_error);
// the GGUF file is not referenced afterwards. Apply and ApplyExpert may be
// called from several threads; the library serialises them.
namespace gufo_npu::cuda {

class CudaProjections : public qwen35::Projections {
public:
  explicit CudaProjections(const gguf::File& file, int device = 0);
  ~CudaProjections() override;
  CudaProjections(const CudaProjections&) = delete;
  CudaProjections& operator=(const CudaProjections&) = delete;

  void Apply(qwen35::Stage stage, int layer, const float* x, int tokens,
             float* y) const override;
  void ApplyExpert(qwen35::Stage stage, int layer, int expert, const float* x,
                   int tokens, float* y) const override;

  gufo_cuda_ctx* context() const { return ctx_; }

  // Matrix handles of one layer, for the device-resident decoder
  // (cuda_decoder.hpp): the input product's parts in stage order, the output
  // matrix, the FFN (dense or shared expert) and, for MoE layers, the router
  // rows and the stacked expert tensors.
  struct LayerHandles {
    long long in[4] = {0, 0, 0, 0};
    long long out = 0;
    long long ffn_gate = 0, ffn_up = 0, ffn_down = 0;
    long long router[2] = {0, 0};
    long long gate_exps = 0, up_exps = 0, down_exps = 0;
  };
  LayerHandles Handles(int layer) const;
  long long HeadHandle() const { return lm_head_.w; }
  // The embedding matrix: the LM head when the embeddings are tied, uploaded on
  // first use otherwise.
  long long EmbeddingHandle(const gguf::File& file) const;

  // Rows [first, first + rows) of an uploaded matrix.
  struct Rows {
    long long w = 0;
    long long first = 0;
    long long rows = 0;
  };

private:
  struct Layer;
  void MatMul(const std::vector<Rows>& parts, const float* x, int tokens,
              float* y) const;
  Rows Upload(const gguf::TensorInfo& t) const;

  qwen35::Config config_;
  gufo_cuda_ctx* ctx_ = nullptr;
  std::vector<Layer> layers_;
  Rows lm_head_;
  mutable Rows embedding_;
};

}  // namespace gufo_npu::cuda
