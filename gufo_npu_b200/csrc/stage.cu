// Staging of fp32 activations into the fixed-point image the tensor-core GEMV
// kernels multiply against (layout and rationale in mma_common.cuh).
//
// One warp converts one 256-value block of one token: every lane takes eight
// adjacent values, the block's largest magnitude fixes the shift, and the three
// signed byte planes, the per-group fp32 sums and the per-column scale factors
// are written to the context's image buffer. The work is a few kilobytes; the
// kernel exists so that this conversion happens once per product and not once
// per thread block of the GEMV.
#include "mma_common.cuh"

namespace gufo {
namespace {

struct StageArgs {
  const float* x;
  uint8_t* image;
  ImageLayout layout;
  float extra;
};

__global__ void __launch_bounds__(kFastThreads)
StageKernel(const __grid_constant__ StageArgs a) {
  const ImageLayout& l = a.layout;
  const int lane = threadIdx.x & 31;
  const int blocks = l.cols / kSuperBlock;
  const int item = blockIdx.x * kFastWarps + (threadIdx.x >> 5);
  GridLaunchDependents();
  GridDependencyWait();
  float* scale = reinterpret_cast<float*>(a.image + l.scale_at);
  if (blockIdx.x == 0) {
    // Columns without a token keep a zero factor.
    for (int i = threadIdx.x; i < blocks * l.kcols; i += kFastThreads) {
      if (i % l.kcols >= l.tokens * kLimbs) {
        scale[i] = 0.f;
      }
    }
  }
  if (item >= l.tokens * blocks) {
    return;
  }
  const int tok = item / blocks;
  const int b = item - tok * blocks;
  const float* xp = a.x + static_cast<size_t>(tok) * l.cols + b * kSuperBlock + lane * 8;
  const float4 v0 = *reinterpret_cast<const float4*>(xp);
  const float4 v1 = *reinterpret_cast<const float4*>(xp + 4);
  const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  StageBlock(v, lane, tok, b, l, a.image, a.extra);
}

}  // namespace

int StageActivations(gufo_cuda_ctx* ctx, const float* x, int tokens, int cols,
                     int group, float extra, const uint8_t** image) {
  StageArgs args;
  args.layout = MakeImageLayout(tokens, cols, group);
  const size_t need = static_cast<size_t>(args.layout.bytes);
  const int grow = ctx->GrowScratch(&ctx->image, &ctx->image_bytes, need, 256u << 10, "staging");
  if (grow != GUFO_CUDA_OK) {
    return grow;
  }
  if (ctx->reuse_image) {
    *image = ctx->image;
    return GUFO_CUDA_OK;
  }
  args.x = x;
  args.image = ctx->image;
  args.extra = extra;
  const int items = tokens * (cols / kSuperBlock);
  const int grid = (items + kFastWarps - 1) / kFastWarps;
  GUFO_CUDA_TRY(LaunchOverlapped(StageKernel, dim3(grid), dim3(kFastThreads), 0, ctx->stream, 1, args));
  ctx->launches.fetch_add(1);
  *image = ctx->image;
  return GUFO_CUDA_OK;
}

// ---- a product that allocates nothing ---------------------------------------

// The staging buffer of gufo_cuda_matmul_q4k_static_device: part of the loaded
// library's image on every GPU that loads it, until the process exits.
constexpr int kStaticImageBytes = 64 * 1024;
static __device__ __align__(256) uint8_t g_static_image[kStaticImageBytes];

namespace {

// Device address of g_static_image per device ordinal, looked up once per
// device: in host code the array's name is only a handle for the runtime, not
// an address a kernel could use.
uint8_t* g_static_image_address[64] = {};
std::mutex g_static_image_mutex;

int StaticImageAddress(int device, uint8_t** out) {
  if (device < 0 || device >= 64) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_q4k_static: device ordinal out of range");
  }
  std::lock_guard<std::mutex> lock(g_static_image_mutex);
  if (g_static_image_address[device] == nullptr) {
    void* address = nullptr;
    GUFO_CUDA_TRY(cudaGetSymbolAddress(&address, g_static_image));
    g_static_image_address[device] = static_cast<uint8_t*>(address);
  }
  *out = g_static_image_address[device];
  return GUFO_CUDA_OK;
}

}  // namespace
}  // namespace gufo

extern "C" int gufo_cuda_matmul_q4k_static_device(gufo_cuda_ctx* ctx, const void* device_weights,
                                                  int64_t rows, int64_t cols, const float* device_x,
                                                  int tokens, float* device_y) {
  using gufo::Fail;
  if (ctx == nullptr || device_weights == nullptr || device_x == nullptr || device_y == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_q4k_static: null pointer");
  }
  if (rows <= 0 || rows > INT32_MAX || cols <= 0 || cols % gufo::kSuperBlock != 0 || tokens < 1 ||
      tokens > gufo::kMaxTokensFast) {
    return Fail(GUFO_CUDA_SHAPE, "matmul_q4k_static: rows > 0, cols a multiple of 256, 1 to 8 tokens");
  }
  if (reinterpret_cast<uintptr_t>(device_weights) % 16 != 0 || reinterpret_cast<uintptr_t>(device_x) % 16 != 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matmul_q4k_static: weights and x must be 16-byte aligned");
  }
  // Three byte planes per token: no row wider than this can fit, and the bound
  // keeps the int arithmetic of the layout below in range.
  if (cols > gufo::kStaticImageBytes / gufo::kLimbs) {
    return Fail(GUFO_CUDA_TOO_LARGE, "matmul_q4k_static: rows of " + std::to_string(cols) +
                                         " values cannot fit the built-in buffer of " +
                                         std::to_string(gufo::kStaticImageBytes) + " bytes");
  }
  gufo::StageArgs stage;
  stage.layout = gufo::MakeImageLayout(tokens, static_cast<int>(cols), 32);
  if (stage.layout.bytes > gufo::kStaticImageBytes || !gufo::Q4KFastFits(static_cast<int>(cols), tokens)) {
    return Fail(GUFO_CUDA_TOO_LARGE,
                "matmul_q4k_static: the staged activations of " + std::to_string(tokens) + " x " +
                    std::to_string(cols) + " values need " + std::to_string(stage.layout.bytes) +
                    " bytes; the built-in buffer holds " + std::to_string(gufo::kStaticImageBytes));
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  uint8_t* image = nullptr;
  const int rc = gufo::StaticImageAddress(ctx->device, &image);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  // Every byte the product reads from the buffer (planes, column factors,
  // group sums) is rewritten here, so nothing has to start at zero.
  stage.x = device_x;
  stage.image = image;
  stage.extra = 1.0f / 16.0f;
  const int items = tokens * static_cast<int>(cols / gufo::kSuperBlock);
  GUFO_CUDA_TRY(gufo::LaunchOverlapped(gufo::StageKernel, dim3((items + gufo::kFastWarps - 1) / gufo::kFastWarps),
                                       dim3(gufo::kFastThreads), 0, ctx->stream, 1, stage));
  ctx->launches.fetch_add(1);
  const gufo::FastGemvArgs args = gufo::ImageGemvArgs(
      static_cast<const uint8_t*>(device_weights), static_cast<int>(rows), static_cast<int>(cols),
      static_cast<int>(gufo::RowBytes(GUFO_CUDA_Q4_K, cols)), image, device_y, static_cast<int>(rows), 0, tokens);
  return gufo::LaunchGemvQ4KFast(ctx, args);
}
