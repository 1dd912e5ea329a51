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
// projection tensor's shape like GgufProjections and uploads the Q4_K, Q6_K and
// F32 tensors once; the GGUF file is not referenced afterwards. Apply and
// ApplyExpert may be called from several threads; the library serialises them.
// Tensors of other types (Q5_K, Q8_0, F16, BF16) throw std::runtime_error.
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
  Rows Upload(const gguf::TensorInfo& t);

  qwen35::Config config_;
  gufo_cuda_ctx* ctx_ = nullptr;
  std::vector<Layer> layers_;
  Rows lm_head_;
};

}  // namespace gufo_npu::cuda
