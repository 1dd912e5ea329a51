// Step-level drop-in check: TEST INFRASTRUCTURE ONLY.
//
// Runs the reference's own Decoder::Step twice over one GGUF file, once with its
// GgufProjections (fp32) and once with the CUDA adapter
// (integration/src_cuda/cuda_projections.cpp over libgufo_cuda.so) plugged in
// behind the same Projections interface, and compares the logits of every
// step; a third run takes the same tokens through the device-resident
// cuda::Decoder (integration/src_cuda/cuda_decoder.cpp), and a fourth walks them
// in two-token steps whose drafts are kept or rolled back (Step(tokens, count) /
// Resolve), every row against the reference's one-token logits. Built by
// oracle/Makefile from the reference's sources where they lie; the mixers, norms
// and sampling stay the reference's CPU code in the first two runs.
//
//   adapter_parity <model.gguf> <tokens>     exit 0 when every step agrees
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "core/gguf.hpp"
#include "cuda/cuda_decoder.hpp"
#include "cuda/cuda_projections.hpp"
#include "models/qwen35/decoder.hpp"
#include "models/qwen35/gguf_projections.hpp"
#include "models/qwen35/reference.hpp"

int main(int argc, char** argv) {
  if (argc != 3) {
    std::fprintf(stderr, "usage: adapter_parity <model.gguf> <tokens>\n");
    return 2;
  }
  namespace qwen35 = gufo_npu::qwen35;
  const auto file = gufo_npu::gguf::File::Open(argv[1]);
  const int steps = std::atoi(argv[2]);
  qwen35::GgufProjections cpu(*file, qwen35::GgufProjections::Precision::kFloat);
  gufo_npu::cuda::CudaProjections gpu(*file, 0);
  qwen35::Decoder a(*file, cpu);
  qwen35::Decoder b(*file, gpu);
  gufo_npu::cuda::Decoder resident(*file, gpu, steps + 8);
  auto sa = a.NewState();
  auto sb = b.NewState();
  const int vocab = a.config().vocab;
  double worst = 0;
  std::vector<int> tokens;
  std::vector<std::vector<float>> wanted;
  for (int s = 0; s < steps; ++s) {
    const int token = (s * 7919 + 13) % vocab;
    const std::vector<float> want = a.Step(token, sa);
    tokens.push_back(token);
    wanted.push_back(want);
    const std::vector<float>& got = b.Step(token, sb);
    double num = 0, den = 0;
    int arg_want = 0, arg_got = 0;
    for (int i = 0; i < vocab; ++i) {
      num += (double(got[i]) - want[i]) * (double(got[i]) - want[i]);
      den += double(want[i]) * want[i];
      if (want[i] > want[arg_want]) arg_want = i;
      if (got[i] > got[arg_got]) arg_got = i;
    }
    const double err = std::sqrt(num / den);
    worst = err > worst ? err : worst;
    std::printf("step %d: logits rel-L2 %.3e argmax %d/%d\n", s, err, arg_got, arg_want);
    if (err > 2e-3 || arg_want != arg_got) {
      std::printf("FAIL\n");
      return 1;
    }
    // The same token through the device-resident decoder.
    const std::vector<float>& on_device = resident.Step(token);
    double num2 = 0;
    int arg_device = 0;
    for (int i = 0; i < vocab; ++i) {
      num2 += (double(on_device[i]) - want[i]) * (double(on_device[i]) - want[i]);
      if (on_device[i] > on_device[arg_device]) arg_device = i;
    }
    const double err2 = std::sqrt(num2 / den);
    worst = err2 > worst ? err2 : worst;
    std::printf("step %d: resident decoder rel-L2 %.3e argmax %d/%d\n", s, err2, arg_device, arg_want);
    if (err2 > 2e-3 || arg_want != arg_device || resident.position() != s + 1) {
      std::printf("FAIL\n");
      return 1;
    }
  }
  // Two-token steps: pairs alternately kept and rolled back (a rolled-back
  // draft is a wrong token, so the next step must not see any trace of it).
  gufo_npu::cuda::Decoder pairs(*file, gpu, steps + 8);
  auto row_error = [&](const float* got, int s) {
    double num = 0, den = 0;
    for (int i = 0; i < vocab; ++i) {
      num += (double(got[i]) - wanted[s][i]) * (double(got[i]) - wanted[s][i]);
      den += double(wanted[s][i]) * wanted[s][i];
    }
    return std::sqrt(num / den);
  };
  bool keep = true;
  for (int s = 0; s < steps;) {
    if (s + 1 >= steps) {
      const double err = row_error(pairs.Step(&tokens[s], 1), s);
      std::printf("pair walk, step %d alone: rel-L2 %.3e\n", s, err);
      worst = err > worst ? err : worst;
      if (err > 2e-3) {
        std::printf("FAIL\n");
        return 1;
      }
      ++s;
      continue;
    }
    const int pair[2] = {tokens[s], keep ? tokens[s + 1] : (tokens[s + 1] + 7) % vocab};
    const float* both = pairs.Step(pair, 2);
    const double first = row_error(both, s);
    const double second = keep ? row_error(both + vocab, s + 1) : 0.0;
    pairs.Resolve(keep);
    std::printf("pair walk, steps %d+%d %s: rel-L2 %.3e %.3e\n", s, s + 1, keep ? "kept" : "rolled back", first,
                second);
    worst = std::fmax(worst, std::fmax(first, second));
    s += keep ? 2 : 1;
    if (first > 2e-3 || second > 2e-3 || pairs.position() != s) {
      std::printf("FAIL\n");
      return 1;
    }
    keep = !keep;
  }
  // A file with an MTP layer: Stage::kMtpIn and the MTP layer's own stages at
  // layer index `layers`, adapter against GgufProjections on the same rows.
  if (qwen35::HasMtpLayer(*file, a.config())) {
    const qwen35::Config& c = a.config();
    const qwen35::Stage stages[] = {qwen35::Stage::kMtpIn, qwen35::Stage::kAttentionIn, qwen35::Stage::kMixerOut,
                                    qwen35::Stage::kFfnIn, qwen35::Stage::kFfnDown};
    for (const qwen35::Stage stage : stages) {
      const int in = qwen35::StageInputs(c, stage, c.layers);
      const int out = qwen35::StageOutputs(c, stage, c.layers);
      std::vector<float> x(static_cast<std::size_t>(2) * in), want(static_cast<std::size_t>(2) * out),
          got(static_cast<std::size_t>(2) * out);
      for (std::size_t i = 0; i < x.size(); ++i) {
        x[i] = std::sin(0.37 * static_cast<double>(i) + static_cast<int>(stage));
      }
      cpu.Apply(stage, c.layers, x.data(), 2, want.data());
      gpu.Apply(stage, c.layers, x.data(), 2, got.data());
      double num = 0, den = 0;
      for (std::size_t i = 0; i < want.size(); ++i) {
        num += (double(got[i]) - want[i]) * (double(got[i]) - want[i]);
        den += double(want[i]) * want[i];
      }
      const double err = std::sqrt(num / den);
      std::printf("MTP layer, stage %d: rel-L2 %.3e\n", static_cast<int>(stage), err);
      worst = err > worst ? err : worst;
      if (err > 1e-3) {
        std::printf("FAIL\n");
        return 1;
      }
    }
  }
  std::printf("PASS: %d steps, worst rel-L2 %.3e\n", steps, worst);
  return 0;
}
