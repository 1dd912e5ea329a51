#include "cuda/cuda_projections.hpp"

#include <stdexcept>
#include <string>

#include "gufo_cuda.h"

// Binds qwen35::Projections to the C ABI of libgufo_cuda. The stage-to-tensor
// mapping is GgufProjections' (src/models/qwen35/gguf_projections.cpp:100-175);
// the products run on the device.
namespace gufo_npu::cuda {
namespace {

using gguf::TensorInfo;

[[noreturn]] void Throw(gufo_cuda_ctx* ctx, int status) {
  const std::string text = gufo_cuda_last_error(ctx);
  switch (status) {
    case GUFO_CUDA_BAD_ARGUMENT:
      throw std::logic_error("cuda: " + text);
    default:
      throw std::runtime_error("cuda: " + text);
  }
}

void Check(gufo_cuda_ctx* ctx, int status) {
  if (status != GUFO_CUDA_OK) {
    Throw(ctx, status);
  }
}

void CheckShape(const TensorInfo& t, std::uint64_t cols, std::uint64_t rows,
                std::uint64_t experts = 0) {
  std::vector<std::uint64_t> want = {cols, rows};
  if (experts != 0) {
    want.push_back(experts);
  } else if (rows == 1 && t.shape.size() == 1) {
    want.pop_back();
  }
  if (t.shape != want) {
    throw std::runtime_error("qwen35: tensor " + t.name + " has an unexpected shape");
  }
}

}  // namespace

struct CudaProjections::Layer {
  std::vector<Rows> linear_in, attention_in, mixer_out, ffn_in, ffn_down, router;
  Rows gate_exps, up_exps, down_exps;
};

CudaProjections::Rows CudaProjections::Upload(const TensorInfo& t) const {
  gufo_cuda_matrix handle = 0;
  Check(ctx_, gufo_cuda_matrix_upload(ctx_, static_cast<int>(t.type), t.data,
                                      static_cast<long long>(t.Rows()),
                                      static_cast<long long>(t.RowElements()), &handle));
  return {handle, 0, static_cast<long long>(t.Rows())};
}

CudaProjections::CudaProjections(const gguf::File& file, int device)
    : config_(qwen35::ReadConfig(file)) {
  Check(nullptr, gufo_cuda_ctx_create(device, nullptr, &ctx_));
  const qwen35::Config& c = config_;
  const auto& embed = file.Tensor("token_embd.weight");
  const auto& head = c.tied_embeddings ? embed : file.Tensor("output.weight");
  CheckShape(head, c.hidden, c.vocab);
  lm_head_ = Upload(head);
  const auto key_dim = static_cast<std::uint64_t>(c.LinearKeyDim());
  const auto value_dim = static_cast<std::uint64_t>(c.LinearValueDim());
  const auto attn_dim = static_cast<std::uint64_t>(c.heads * c.head_dim);
  const auto kv_dim = static_cast<std::uint64_t>(c.kv_heads * c.head_dim);
  for (int il = 0; il < c.layers; ++il) {
    const std::string p = "blk." + std::to_string(il) + ".";
    auto t = [&](const std::string& name) -> const TensorInfo& { return file.Tensor(p + name); };
    Layer layer;
    if (c.IsMoe()) {
      CheckShape(t("ffn_gate_inp.weight"), c.hidden, c.experts);
      CheckShape(t("ffn_gate_inp_shexp.weight"), c.hidden, 1);
      layer.router = {Upload(t("ffn_gate_inp.weight")), Upload(t("ffn_gate_inp_shexp.weight"))};
      CheckShape(t("ffn_gate_exps.weight"), c.hidden, c.expert_ffn, c.experts);
      CheckShape(t("ffn_up_exps.weight"), c.hidden, c.expert_ffn, c.experts);
      CheckShape(t("ffn_down_exps.weight"), c.expert_ffn, c.hidden, c.experts);
      layer.gate_exps = Upload(t("ffn_gate_exps.weight"));
      layer.up_exps = Upload(t("ffn_up_exps.weight"));
      layer.down_exps = Upload(t("ffn_down_exps.weight"));
    }
    const std::string suffix = c.IsMoe() ? "_shexp.weight" : ".weight";
    CheckShape(t("ffn_gate" + suffix), c.hidden, c.FfnWidth());
    CheckShape(t("ffn_up" + suffix), c.hidden, c.FfnWidth());
    CheckShape(t("ffn_down" + suffix), c.FfnWidth(), c.hidden);
    layer.ffn_in = {Upload(t("ffn_gate" + suffix)), Upload(t("ffn_up" + suffix))};
    layer.ffn_down = {Upload(t("ffn_down" + suffix))};
    if (c.IsFullAttention(il)) {
      CheckShape(t("attn_q.weight"), c.hidden, 2 * attn_dim);
      CheckShape(t("attn_k.weight"), c.hidden, kv_dim);
      CheckShape(t("attn_v.weight"), c.hidden, kv_dim);
      CheckShape(t("attn_output.weight"), attn_dim, c.hidden);
      layer.attention_in = {Upload(t("attn_q.weight")), Upload(t("attn_k.weight")),
                            Upload(t("attn_v.weight"))};
      layer.mixer_out = {Upload(t("attn_output.weight"))};
    } else {
      CheckShape(t("attn_qkv.weight"), c.hidden, 2 * key_dim + value_dim);
      CheckShape(t("attn_gate.weight"), c.hidden, value_dim);
      CheckShape(t("ssm_alpha.weight"), c.hidden, c.linear_value_heads);
      CheckShape(t("ssm_beta.weight"), c.hidden, c.linear_value_heads);
      CheckShape(t("ssm_out.weight"), value_dim, c.hidden);
      layer.linear_in = {Upload(t("attn_qkv.weight")), Upload(t("attn_gate.weight")),
                         Upload(t("ssm_alpha.weight")), Upload(t("ssm_beta.weight"))};
      layer.mixer_out = {Upload(t("ssm_out.weight"))};
    }
    layers_.push_back(std::move(layer));
  }
}

CudaProjections::~CudaProjections() { gufo_cuda_ctx_destroy(ctx_); }

CudaProjections::LayerHandles CudaProjections::Handles(int layer) const {
  const Layer& l = layers_.at(static_cast<std::size_t>(layer));
  LayerHandles h;
  const std::vector<Rows>& in = l.linear_in.empty() ? l.attention_in : l.linear_in;
  for (std::size_t i = 0; i < in.size() && i < 4; ++i) {
    h.in[i] = in[i].w;
  }
  h.out = l.mixer_out.at(0).w;
  h.ffn_gate = l.ffn_in.at(0).w;
  h.ffn_up = l.ffn_in.at(1).w;
  h.ffn_down = l.ffn_down.at(0).w;
  if (!l.router.empty()) {
    h.router[0] = l.router.at(0).w;
    h.router[1] = l.router.at(1).w;
    h.gate_exps = l.gate_exps.w;
    h.up_exps = l.up_exps.w;
    h.down_exps = l.down_exps.w;
  }
  return h;
}

long long CudaProjections::EmbeddingHandle(const gguf::File& file) const {
  if (config_.tied_embeddings) {
    return lm_head_.w;
  }
  if (embedding_.w == 0) {
    embedding_ = Upload(file.Tensor("token_embd.weight"));
  }
  return embedding_.w;
}

void CudaProjections::MatMul(const std::vector<Rows>& parts, const float* x,
                             int tokens, float* y) const {
  std::vector<gufo_cuda_rows> rows;
  for (const auto& part : parts) {
    rows.push_back({part.w, part.first, part.rows});
  }
  Check(ctx_, gufo_cuda_matmul(ctx_, rows.data(), static_cast<int>(rows.size()), x, tokens, y));
}

void CudaProjections::Apply(qwen35::Stage stage, int layer, const float* x,
                            int tokens, float* y) const {
  using qwen35::Stage;
  if (stage == Stage::kLmHead) {
    return MatMul({lm_head_}, x, tokens, y);
  }
  const Layer& l = layers_.at(static_cast<std::size_t>(layer));
  const std::vector<Rows>* parts = nullptr;
  switch (stage) {
    case Stage::kLinearIn: parts = &l.linear_in; break;
    case Stage::kAttentionIn: parts = &l.attention_in; break;
    case Stage::kMixerOut: parts = &l.mixer_out; break;
    case Stage::kFfnIn: parts = &l.ffn_in; break;
    case Stage::kFfnDown: parts = &l.ffn_down; break;
    case Stage::kRouter: parts = &l.router; break;
    default: break;
  }
  if (parts == nullptr || parts->empty()) {
    throw std::logic_error("qwen35: no weights for this stage and layer");
  }
  MatMul(*parts, x, tokens, y);
}

void CudaProjections::ApplyExpert(qwen35::Stage stage, int layer, int expert,
                                  const float* x, int tokens, float* y) const {
  using qwen35::Stage;
  const Layer& l = layers_.at(static_cast<std::size_t>(layer));
  if (l.gate_exps.w == 0 || expert < 0 || expert >= config_.experts) {
    throw std::logic_error("qwen35: no such expert");
  }
  const long long e = expert;
  const long long ffn = config_.expert_ffn;
  const long long hidden = config_.hidden;
  switch (stage) {
    case Stage::kExpertIn:
      return MatMul({{l.gate_exps.w, e * ffn, ffn}, {l.up_exps.w, e * ffn, ffn}}, x, tokens, y);
    case Stage::kExpertDown:
      return MatMul({{l.down_exps.w, e * hidden, hidden}}, x, tokens, y);
    default:
      throw std::logic_error("qwen35: ApplyExpert takes expert stages only");
  }
}

}  // namespace gufo_npu::cuda
