#include "cuda/cuda_projections.hpp"

#include <stdexcept>
#include <string>

#include "gufo_cuda.h"

// Binds qwen35::Projections to the C ABI of libgufo_cuda. The stage-to-tensor
// mapping is GgufProjections' (src/models/qwen35/gguf_projections.cpp:100-175),
// written here as one table; the products run on the device.
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

// One row of the stage table: a tensor of a layer, the stage whose product it
// joins (in table order), and its shape [cols, rows (, experts)] in terms of
// the model's widths. The table is the whole of the mapping
// (src/models/qwen35/gguf_projections.cpp:114-171 builds the same lists).
enum class Width { kHidden, kTwoHidden, kFfn, kAttn, kTwoAttn, kKv, kConv, kValue, kValueHeads, kExperts, kExpertFfn, kOne };
enum class When { kAlways, kMoe, kAttention, kLinear, kMtp };
struct StageTensor {
  qwen35::Stage stage;
  const char* name;       // "%" stands for "_shexp" in MoE models and for nothing otherwise
  Width cols, rows;
  bool stacked;           // a third dimension of `experts` matrices
  When when;
};
constexpr StageTensor kStageTable[] = {
    {qwen35::Stage::kMtpIn, "nextn.eh_proj.weight", Width::kTwoHidden, Width::kHidden, false, When::kMtp},
    {qwen35::Stage::kRouter, "ffn_gate_inp.weight", Width::kHidden, Width::kExperts, false, When::kMoe},
    {qwen35::Stage::kRouter, "ffn_gate_inp_shexp.weight", Width::kHidden, Width::kOne, false, When::kMoe},
    {qwen35::Stage::kExpertIn, "ffn_gate_exps.weight", Width::kHidden, Width::kExpertFfn, true, When::kMoe},
    {qwen35::Stage::kExpertIn, "ffn_up_exps.weight", Width::kHidden, Width::kExpertFfn, true, When::kMoe},
    {qwen35::Stage::kExpertDown, "ffn_down_exps.weight", Width::kExpertFfn, Width::kHidden, true, When::kMoe},
    {qwen35::Stage::kFfnIn, "ffn_gate%.weight", Width::kHidden, Width::kFfn, false, When::kAlways},
    {qwen35::Stage::kFfnIn, "ffn_up%.weight", Width::kHidden, Width::kFfn, false, When::kAlways},
    {qwen35::Stage::kFfnDown, "ffn_down%.weight", Width::kFfn, Width::kHidden, false, When::kAlways},
    {qwen35::Stage::kAttentionIn, "attn_q.weight", Width::kHidden, Width::kTwoAttn, false, When::kAttention},
    {qwen35::Stage::kAttentionIn, "attn_k.weight", Width::kHidden, Width::kKv, false, When::kAttention},
    {qwen35::Stage::kAttentionIn, "attn_v.weight", Width::kHidden, Width::kKv, false, When::kAttention},
    {qwen35::Stage::kMixerOut, "attn_output.weight", Width::kAttn, Width::kHidden, false, When::kAttention},
    {qwen35::Stage::kLinearIn, "attn_qkv.weight", Width::kHidden, Width::kConv, false, When::kLinear},
    {qwen35::Stage::kLinearIn, "attn_gate.weight", Width::kHidden, Width::kValue, false, When::kLinear},
    {qwen35::Stage::kLinearIn, "ssm_alpha.weight", Width::kHidden, Width::kValueHeads, false, When::kLinear},
    {qwen35::Stage::kLinearIn, "ssm_beta.weight", Width::kHidden, Width::kValueHeads, false, When::kLinear},
    {qwen35::Stage::kMixerOut, "ssm_out.weight", Width::kValue, Width::kHidden, false, When::kLinear},
};

std::uint64_t WidthOf(const qwen35::Config& c, Width w) {
  switch (w) {
    case Width::kHidden: return static_cast<std::uint64_t>(c.hidden);
    case Width::kTwoHidden: return 2 * static_cast<std::uint64_t>(c.hidden);
    case Width::kFfn: return static_cast<std::uint64_t>(c.FfnWidth());
    case Width::kAttn: return static_cast<std::uint64_t>(c.heads * c.head_dim);
    case Width::kTwoAttn: return 2 * static_cast<std::uint64_t>(c.heads * c.head_dim);
    case Width::kKv: return static_cast<std::uint64_t>(c.kv_heads * c.head_dim);
    case Width::kConv: return static_cast<std::uint64_t>(c.ConvChannels());
    case Width::kValue: return static_cast<std::uint64_t>(c.LinearValueDim());
    case Width::kValueHeads: return static_cast<std::uint64_t>(c.linear_value_heads);
    case Width::kExperts: return static_cast<std::uint64_t>(c.experts);
    case Width::kExpertFfn: return static_cast<std::uint64_t>(c.expert_ffn);
    case Width::kOne: return 1;
  }
  return 0;
}

constexpr int kStages = static_cast<int>(qwen35::Stage::kMtpIn) + 1;

}  // namespace

// Per layer and stage, the uploaded tensors in table order.
struct CudaProjections::Layer {
  std::vector<Rows> parts[kStages];
  const std::vector<Rows>& of(qwen35::Stage stage) const { return parts[static_cast<int>(stage)]; }
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
  if (head.shape != std::vector<std::uint64_t>{static_cast<std::uint64_t>(c.hidden), static_cast<std::uint64_t>(c.vocab)}) {
    throw std::runtime_error("qwen35: tensor " + head.name + " has an unexpected shape");
  }
  lm_head_ = Upload(head);
  // The decoder layers, then the MTP layer (full attention) if present.
  const int loaded = c.layers + (qwen35::HasMtpLayer(file, c) ? 1 : 0);
  for (int il = 0; il < loaded; ++il) {
    const std::string p = "blk." + std::to_string(il) + ".";
    Layer layer;
    for (const StageTensor& row : kStageTable) {
      const bool wanted = row.when == When::kAlways || (row.when == When::kMoe && c.IsMoe()) ||
                          (row.when == When::kAttention && c.IsFullAttention(il)) ||
                          (row.when == When::kLinear && !c.IsFullAttention(il)) ||
                          (row.when == When::kMtp && il >= c.layers);
      if (!wanted) {
        continue;
      }
      std::string name = row.name;
      const auto mark = name.find('%');
      if (mark != std::string::npos) {
        name.replace(mark, 1, c.IsMoe() ? "_shexp" : "");
      }
      const TensorInfo& t = file.Tensor(p + name);
      std::vector<std::uint64_t> want = {WidthOf(c, row.cols), WidthOf(c, row.rows)};
      if (row.stacked) {
        want.push_back(static_cast<std::uint64_t>(c.experts));
      } else if (want[1] == 1 && t.shape.size() == 1) {
        want.pop_back();
      }
      if (t.shape != want) {
        throw std::runtime_error("qwen35: tensor " + t.name + " has an unexpected shape");
      }
      layer.parts[static_cast<int>(row.stage)].push_back(Upload(t));
    }
    layers_.push_back(std::move(layer));
  }
}

CudaProjections::~CudaProjections() { gufo_cuda_ctx_destroy(ctx_); }

CudaProjections::LayerHandles CudaProjections::Handles(int layer) const {
  using qwen35::Stage;
  const Layer& l = layers_.at(static_cast<std::size_t>(layer));
  LayerHandles h;
  const std::vector<Rows>& in = l.of(Stage::kLinearIn).empty() ? l.of(Stage::kAttentionIn) : l.of(Stage::kLinearIn);
  for (std::size_t i = 0; i < in.size() && i < 4; ++i) {
    h.in[i] = in[i].w;
  }
  h.out = l.of(Stage::kMixerOut).at(0).w;
  h.ffn_gate = l.of(Stage::kFfnIn).at(0).w;
  h.ffn_up = l.of(Stage::kFfnIn).at(1).w;
  h.ffn_down = l.of(Stage::kFfnDown).at(0).w;
  if (!l.of(Stage::kRouter).empty()) {
    h.router[0] = l.of(Stage::kRouter).at(0).w;
    h.router[1] = l.of(Stage::kRouter).at(1).w;
    h.gate_exps = l.of(Stage::kExpertIn).at(0).w;
    h.up_exps = l.of(Stage::kExpertIn).at(1).w;
    h.down_exps = l.of(Stage::kExpertDown).at(0).w;
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
  // The stacked expert tensors are reached through ApplyExpert only.
  if (stage == Stage::kExpertIn || stage == Stage::kExpertDown || l.of(stage).empty()) {
    throw std::logic_error("qwen35: no weights for this stage and layer");
  }
  MatMul(l.of(stage), x, tokens, y);
}

void CudaProjections::ApplyExpert(qwen35::Stage stage, int layer, int expert,
                                  const float* x, int tokens, float* y) const {
  using qwen35::Stage;
  const Layer& l = layers_.at(static_cast<std::size_t>(layer));
  if (l.of(Stage::kExpertIn).empty() || expert < 0 || expert >= config_.experts) {
    throw std::logic_error("qwen35: no such expert");
  }
  if (stage != Stage::kExpertIn && stage != Stage::kExpertDown) {
    throw std::logic_error("qwen35: ApplyExpert takes expert stages only");
  }
  // Expert e is a row slice of every stacked tensor of the stage: rows
  // [e * n, (e + 1) * n) with n the rows of one expert's matrix.
  std::vector<Rows> parts;
  for (const Rows& all : l.of(stage)) {
    const long long n = all.rows / config_.experts;
    parts.push_back({all.w, expert * n, n});
  }
  MatMul(parts, x, tokens, y);
}

}  // namespace gufo_npu::cuda
