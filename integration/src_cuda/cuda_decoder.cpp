#include "cuda/cuda_decoder.hpp"

#include <stdexcept>
#include <string>

#include "core/quant.hpp"
#include "gufo_cuda.h"
#include "models/qwen35/config.hpp"

// Binds the device-resident decode step of libgufo_cuda (gufo_cuda_decoder_*)
// to a class shaped like qwen35::Decoder. The small fp32 vectors are read from
// the GGUF file the way Decoder and Mixer read them
// (src/models/qwen35/decoder.cpp:19-23,73-87,447-455).
namespace gufo_npu::cuda {
namespace {

std::vector<float> ToFloats(const gguf::TensorInfo& t) {
  std::vector<float> out(t.num_elements);
  quant::Dequantize(t.type, t.data, out.data(), out.size());
  return out;
}

}  // namespace

Decoder::Decoder(const gguf::File& file, const CudaProjections& projections, int max_positions)
    : projections_(projections) {
  const qwen35::Config c = qwen35::ReadConfig(file);
  gufo_cuda_decoder_config config = {};
  config.layers = c.layers;
  config.hidden = c.hidden;
  config.ffn = c.FfnWidth();
  config.vocab = c.vocab;
  config.rms_eps = c.rms_eps;
  config.full_attention_interval = c.full_attention_interval;
  config.heads = c.heads;
  config.kv_heads = c.kv_heads;
  config.head_dim = c.head_dim;
  config.rope_dim = c.rope_dim;
  config.rope_theta = c.rope_theta;
  config.conv_kernel = c.conv_kernel;
  config.linear_key_heads = c.linear_key_heads;
  config.linear_value_heads = c.linear_value_heads;
  config.linear_head_dim = c.linear_head_dim;
  config.max_positions = max_positions;
  config.use_graph = 1;
  config.experts = c.experts;
  config.experts_used = c.experts_used;
  config.expert_ffn = c.expert_ffn;

  // The vectors must stay alive until decoder_create has copied them.
  std::vector<std::vector<float>> keep;
  auto vector = [&](const std::string& name) -> const float* {
    keep.push_back(ToFloats(file.Tensor(name)));
    return keep.back().data();
  };
  std::vector<gufo_cuda_layer_weights> layers(static_cast<std::size_t>(c.layers));
  for (int il = 0; il < c.layers; ++il) {
    const std::string p = "blk." + std::to_string(il) + ".";
    gufo_cuda_layer_weights& w = layers[static_cast<std::size_t>(il)];
    w = {};
    const CudaProjections::LayerHandles h = projections.Handles(il);
    w.attn_norm = vector(p + "attn_norm.weight");
    w.post_attention_norm = vector(p + "post_attention_norm.weight");
    if (c.IsFullAttention(il)) {
      w.attn_q = h.in[0];
      w.attn_k = h.in[1];
      w.attn_v = h.in[2];
      w.attn_output = h.out;
      w.attn_q_norm = vector(p + "attn_q_norm.weight");
      w.attn_k_norm = vector(p + "attn_k_norm.weight");
    } else {
      w.attn_qkv = h.in[0];
      w.attn_gate = h.in[1];
      w.ssm_alpha = h.in[2];
      w.ssm_beta = h.in[3];
      w.ssm_out = h.out;
      w.ssm_conv1d = vector(p + "ssm_conv1d.weight");
      w.ssm_a = vector(p + "ssm_a");
      w.ssm_dt_bias = vector(p + "ssm_dt.bias");
      w.ssm_norm = vector(p + "ssm_norm.weight");
    }
    w.ffn_gate = h.ffn_gate;
    w.ffn_up = h.ffn_up;
    w.ffn_down = h.ffn_down;
    if (c.IsMoe()) {
      w.ffn_gate_inp = h.router[0];
      w.ffn_gate_inp_shexp = h.router[1];
      w.ffn_gate_exps = h.gate_exps;
      w.ffn_up_exps = h.up_exps;
      w.ffn_down_exps = h.down_exps;
    }
  }
  gufo_cuda_decoder_weights weights = {};
  weights.token_embd = projections.EmbeddingHandle(file);
  weights.output = c.tied_embeddings ? 0 : projections.HeadHandle();
  weights.output_norm = vector("output_norm.weight");
  weights.layers = layers.data();
  const int status = gufo_cuda_decoder_create(projections.context(), &config, &weights, &decoder_);
  if (status != GUFO_CUDA_OK) {
    throw std::runtime_error(std::string("cuda: ") + gufo_cuda_last_error(projections.context()));
  }
  logits_.resize(static_cast<std::size_t>(c.vocab));
  pair_logits_.resize(2 * logits_.size());
  hidden_width_ = c.hidden;
}

Decoder::~Decoder() { gufo_cuda_decoder_destroy(decoder_); }

const std::vector<float>& Decoder::Step(int token) {
  const int status = gufo_cuda_decoder_step(decoder_, token, logits_.data());
  if (status == GUFO_CUDA_TOO_LARGE) {
    throw std::length_error("cuda: the attention cache is full");
  }
  if (status != GUFO_CUDA_OK) {
    // A bad argument is a token id out of range (Decoder::Step's std::out_of_range,
    // src/models/qwen35/decoder.cpp:483-485) only when the message says so; a step
    // that awaits Resolve is a misuse of the interface.
    const std::string text = gufo_cuda_last_error(projections_.context());
    if (status == GUFO_CUDA_BAD_ARGUMENT) {
      if (text.find("out of range") != std::string::npos) {
        throw std::out_of_range(text);
      }
      throw std::logic_error("cuda: " + text);
    }
    throw std::runtime_error("cuda: " + text);
  }
  return logits_;
}

const float* Decoder::Step(const int* tokens, int count, bool logits) {
  if (count < 1 || count > 2) {
    throw std::invalid_argument("cuda decoder: 1 or 2 tokens per step");
  }
  const int status =
      gufo_cuda_decoder_step_tokens(decoder_, tokens, count, logits ? 1 : 0, logits ? pair_logits_.data() : nullptr);
  if (status == GUFO_CUDA_TOO_LARGE) {
    throw std::length_error("cuda: the attention cache is full");
  }
  if (status != GUFO_CUDA_OK) {
    const std::string text = gufo_cuda_last_error(projections_.context());
    if (status == GUFO_CUDA_BAD_ARGUMENT) {
      if (text.find("out of range") != std::string::npos) {
        throw std::out_of_range(text);
      }
      throw std::logic_error("cuda: " + text);
    }
    throw std::runtime_error("cuda: " + text);
  }
  return logits ? pair_logits_.data() : nullptr;
}

void Decoder::Resolve(bool keep_second) {
  if (gufo_cuda_decoder_resolve(decoder_, keep_second ? 1 : 0) != GUFO_CUDA_OK) {
    throw std::logic_error(std::string("cuda: ") + gufo_cuda_last_error(projections_.context()));
  }
}

const std::vector<float>& Decoder::hidden(int t) {
  const float* device = nullptr;
  hidden_.resize(static_cast<std::size_t>(hidden_width_));
  if (gufo_cuda_decoder_hidden_device(decoder_, t, &device) != GUFO_CUDA_OK ||
      gufo_cuda_download(projections_.context(), hidden_.data(), device, hidden_.size() * sizeof(float)) !=
          GUFO_CUDA_OK) {
    throw std::runtime_error(std::string("cuda: ") + gufo_cuda_last_error(projections_.context()));
  }
  return hidden_;
}

void Decoder::Reset() {
  if (gufo_cuda_decoder_reset(decoder_) != GUFO_CUDA_OK) {
    throw std::runtime_error(std::string("cuda: ") + gufo_cuda_last_error(projections_.context()));
  }
}

int Decoder::position() const { return gufo_cuda_decoder_position(decoder_); }

}  // namespace gufo_npu::cuda
