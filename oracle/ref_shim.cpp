// C entry points over the reference's own CPU sources: TEST INFRASTRUCTURE ONLY.
//
// Built by oracle/Makefile together with the reference's unmodified source
// files (compiled where they lie, by include path) into oracle/_ref/
// libgufo_ref.so. It pins the C restatement in gufo_oracle.c and serves as the
// timed CPU baseline. The product library never links or loads it.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <exception>
#include <memory>
#include <string>
#include <vector>

#include "core/cpus.hpp"
#include "core/gguf.hpp"
#include "core/quant.hpp"
#include "models/qwen35/decoder.hpp"
#include "models/qwen35/gguf_dot.hpp"
#include "models/qwen35/gguf_projections.hpp"
#include "models/qwen35/moe.hpp"
#include "models/qwen35/projections.hpp"
#include "models/qwen35/reference.hpp"
#include "models/qwen35_2b/deltanet.hpp"

namespace {

using namespace gufo_npu;

thread_local std::string g_error;

// A reference model over an in-memory GGUF image.
struct Model {
  std::vector<std::uint8_t> bytes;
  std::unique_ptr<gguf::File> file;
  std::unique_ptr<qwen35::GgufProjections> projections;
  std::unique_ptr<qwen35::Mixer> mixer;
  std::unique_ptr<qwen35::Decoder> decoder;
  std::unique_ptr<qwen35_2b::DeltaNetStep> fused;
  qwen35::DecodeState state;
  bool has_state = false;
};

template <typename F>
int Guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  } catch (...) {
    g_error = "unknown exception";
    return -1;
  }
}

// A DecodeState::Layer around caller-owned flat arrays.
struct LayerView {
  qwen35::DecodeState::Layer layer;
  float* conv;
  float* ssm;
  LayerView(const qwen35::Config& c, float* conv_in, float* ssm_in)
      : conv(conv_in), ssm(ssm_in) {
    const std::size_t conv_n =
        static_cast<std::size_t>(c.conv_kernel - 1) * c.ConvChannels();
    const std::size_t ssm_n = static_cast<std::size_t>(c.linear_value_heads) *
                              c.linear_head_dim * c.linear_head_dim;
    layer.conv.assign(conv, conv + conv_n);
    layer.ssm.assign(ssm, ssm + ssm_n);
  }
  void Store() {
    std::copy(layer.conv.begin(), layer.conv.end(), conv);
    std::copy(layer.ssm.begin(), layer.ssm.end(), ssm);
  }
};

}  // namespace

extern "C" {

const char* gufo_ref_last_error() { return g_error.c_str(); }

int gufo_ref_usable_cpus() { return static_cast<int>(UsableCpus()); }
int gufo_ref_projection_threads() {
  return static_cast<int>(HalfCpuWorkers() + 1);
}

float gufo_ref_half_to_float(std::uint16_t h) { return quant::HalfToFloat(h); }

void gufo_ref_scale_min_k4(std::size_t j, const std::uint8_t* q,
                           std::uint8_t* scale, std::uint8_t* min) {
  quant::ScaleMinK4(j, q, scale, min);
}

int gufo_ref_dequantize(std::uint32_t type, const std::uint8_t* src, float* dst,
                        std::size_t n) {
  return Guard([&] {
    quant::Dequantize(static_cast<gguf::GgmlType>(type), src, dst, n);
  });
}

// The reference's fused fp32 row dot for `type` (AVX2 body in this build).
int gufo_ref_dot(std::uint32_t type, const std::uint8_t* row, const float* x,
                 std::size_t n, float* out) {
  namespace dot = qwen35::gguf_dot;
  switch (static_cast<gguf::GgmlType>(type)) {
    case gguf::GgmlType::kQ8_0:
      *out = dot::DotQ8_0(row, x, n);
      return 0;
    case gguf::GgmlType::kQ4_K:
      *out = dot::DotQ4_K(row, x, n);
      return 0;
    case gguf::GgmlType::kQ5_K:
      *out = dot::DotQ5_K(row, x, n);
      return 0;
    case gguf::GgmlType::kQ6_K:
      *out = dot::DotQ6_K(row, x, n);
      return 0;
    case gguf::GgmlType::kF32:
      *out = dot::DotF32(row, x, n);
      return 0;
    default:
      g_error = "no fused dot for this type";
      return -1;
  }
}

void gufo_ref_route(const float* logits, int experts, int k, int* chosen,
                    float* weights) {
  qwen35::Route(logits, experts, k, chosen, weights);
}

float gufo_ref_shared_expert_scale(float logit) {
  return qwen35::SharedExpertScale(logit);
}

// precision: 0 = GgufProjections::Precision::kDouble, 1 = kFloat.
void* gufo_ref_model_open(const std::uint8_t* bytes, std::size_t size,
                          int precision) {
  auto model = std::make_unique<Model>();
  const int rc = Guard([&] {
    model->bytes.assign(bytes, bytes + size);
    model->file =
        gguf::File::FromBytes(model->bytes.data(), model->bytes.size());
    model->projections = std::make_unique<qwen35::GgufProjections>(
        *model->file, precision == 0
                          ? qwen35::GgufProjections::Precision::kDouble
                          : qwen35::GgufProjections::Precision::kFloat);
    model->mixer = std::make_unique<qwen35::Mixer>(*model->file);
  });
  return rc == 0 ? model.release() : nullptr;
}

void gufo_ref_model_close(void* handle) { delete static_cast<Model*>(handle); }

std::size_t gufo_ref_stage_inputs(void* handle, int stage, int layer) {
  auto* m = static_cast<Model*>(handle);
  return qwen35::StageInputs(m->mixer->config(),
                             static_cast<qwen35::Stage>(stage), layer);
}

std::size_t gufo_ref_stage_outputs(void* handle, int stage, int layer) {
  auto* m = static_cast<Model*>(handle);
  return qwen35::StageOutputs(m->mixer->config(),
                              static_cast<qwen35::Stage>(stage), layer);
}

int gufo_ref_apply(void* handle, int stage, int layer, const float* x,
                   int tokens, float* y) {
  auto* m = static_cast<Model*>(handle);
  return Guard([&] {
    m->projections->Apply(static_cast<qwen35::Stage>(stage), layer, x, tokens,
                          y);
  });
}

int gufo_ref_apply_expert(void* handle, int stage, int layer, int expert,
                          const float* x, int tokens, float* y) {
  auto* m = static_cast<Model*>(handle);
  return Guard([&] {
    m->projections->ApplyExpert(static_cast<qwen35::Stage>(stage), layer,
                                expert, x, tokens, y);
  });
}

// Mixer::Linear on caller-owned state arrays: conv [kernel - 1][channels] and
// ssm [heads][dk][dk] advance in place (ssm stays when ssm_out is given).
int gufo_ref_linear(void* handle, int layer, const float* in, float* conv,
                    float* ssm, float* y, float* ssm_out) {
  auto* m = static_cast<Model*>(handle);
  return Guard([&] {
    LayerView view(m->mixer->config(), conv, ssm);
    m->mixer->Linear(layer, in, view.layer, y, ssm_out);
    view.Store();
  });
}

// DeltaNetStep::Run for `count` (1 or 2) tokens on caller-owned arrays. With
// two tokens ssm_spec and conv_saved (same sizes as ssm and conv) receive the
// speculative state and the saved window.
int gufo_ref_deltanet_run(void* handle, int layer, int count, const float* in,
                          std::size_t in_stride, const float* h,
                          std::size_t h_stride, float* conv, float* ssm,
                          float* ssm_spec, float* conv_saved, float* y,
                          std::size_t y_stride) {
  auto* m = static_cast<Model*>(handle);
  return Guard([&] {
    const auto& c = m->mixer->config();
    if (!m->fused) {
      m->fused = std::make_unique<qwen35_2b::DeltaNetStep>(*m->file, c,
                                                           m->mixer->pool());
    }
    LayerView view(c, conv, ssm);
    m->fused->Run(layer, count, in, in_stride, h, h_stride, view.layer, y,
                  y_stride);
    view.Store();
    if (count == 2) {
      std::copy(view.layer.ssm_spec.begin(), view.layer.ssm_spec.end(),
                ssm_spec);
      std::copy(view.layer.conv_saved.begin(), view.layer.conv_saved.end(),
                conv_saved);
    }
  });
}

// Decoder::Step over the model's own GgufProjections. The state is kept in
// the handle; reset starts a new sequence.
int gufo_ref_decoder_reset(void* handle) {
  auto* m = static_cast<Model*>(handle);
  return Guard([&] {
    if (!m->decoder) {
      m->decoder =
          std::make_unique<qwen35::Decoder>(*m->file, *m->projections);
    }
    m->state = m->decoder->NewState();
    m->has_state = true;
  });
}

int gufo_ref_decoder_step(void* handle, int token, float* logits) {
  auto* m = static_cast<Model*>(handle);
  return Guard([&] {
    if (!m->has_state) {
      throw std::logic_error("decoder_reset first");
    }
    const auto& out = m->decoder->Step(token, m->state);
    if (logits != nullptr) {
      std::copy(out.begin(), out.end(), logits);
    }
  });
}

// Copies layer `il`'s DeltaNet state out of the decoder's sequence state.
int gufo_ref_decoder_linear_state(void* handle, int il, float* conv,
                                  float* ssm) {
  auto* m = static_cast<Model*>(handle);
  return Guard([&] {
    const auto& layer = m->state.layers.at(static_cast<std::size_t>(il));
    std::copy(layer.conv.begin(), layer.conv.end(), conv);
    std::copy(layer.ssm.begin(), layer.ssm.end(), ssm);
  });
}

int gufo_ref_decoder_position(void* handle) {
  return static_cast<Model*>(handle)->state.position;
}

}  // extern "C"
