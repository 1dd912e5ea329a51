#include "cuda/cuda_decoder.hpp"
#include "cuda/cuda_projections.hpp"

#include <stdexcept>

// Built when GUFO_NPU_ENABLE_CUDA is off: the same header, every entry point
// reports that the backend is absent (the pattern of src/npu/gemv_stub.cpp).
namespace gufo_npu::cuda {

struct CudaProjections::Layer {};

CudaProjections::CudaProjections(const gguf::File& file, int)
    : config_(qwen35::ReadConfig(file)) {
  throw std::runtime_error("gufo-npu was built without CUDA");
}
CudaProjections::~CudaProjections() = default;
void CudaProjections::Apply(qwen35::Stage, int, const float*, int, float*) const {
  throw std::runtime_error("gufo-npu was built without CUDA");
}
void CudaProjections::ApplyExpert(qwen35::Stage, int, int, const float*, int, float*) const {
  throw std::runtime_error("gufo-npu was built without CUDA");
}
void CudaProjections::MatMul(const std::vector<Rows>&, const float*, int, float*) const {}
CudaProjections::Rows CudaProjections::Upload(const gguf::TensorInfo&) const { return {}; }
CudaProjections::LayerHandles CudaProjections::Handles(int) const { return {}; }
long long CudaProjections::EmbeddingHandle(const gguf::File&) const { return 0; }

Decoder::Decoder(const gguf::File&, const CudaProjections& projections, int) : projections_(projections) {
  throw std::runtime_error("gufo-npu was built without CUDA");
}
Decoder::~Decoder() = default;
const std::vector<float>& Decoder::Step(int) { throw std::runtime_error("gufo-npu was built without CUDA"); }
const float* Decoder::Step(const int*, int, bool) { throw std::runtime_error("gufo-npu was built without CUDA"); }
void Decoder::Resolve(bool) { throw std::runtime_error("gufo-npu was built without CUDA"); }
const std::vector<float>& Decoder::hidden(int) { throw std::runtime_error("gufo-npu was built without CUDA"); }
void Decoder::Reset() { throw std::runtime_error("gufo-npu was built without CUDA"); }
int Decoder::position() const { return 0; }

}  // namespace gufo_npu::cuda
