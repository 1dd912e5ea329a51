// Context, device memory and weight handles of the C ABI (include/gufo_cuda.h).
#include "common.cuh"
#include "gemm_tc.cuh"

#include <cstring>
#include <new>

namespace gufo {

namespace {
thread_local std::string g_last_error;
}

void SetError(const std::string& text) { g_last_error = text; }

int Fail(int status, const std::string& text) {
  g_last_error = text;
  return status;
}

int CudaFail(cudaError_t e, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return e == cudaErrorMemoryAllocation ? GUFO_CUDA_OUT_OF_MEMORY
                                        : GUFO_CUDA_RUNTIME;
}

size_t RowBytes(int type, int64_t cols) {
  if (cols <= 0) {
    return 0;
  }
  switch (type) {
    case GUFO_CUDA_F32:
      return static_cast<size_t>(cols) * 4;
    case GUFO_CUDA_Q4_K:
      return cols % kSuperBlock ? 0 : static_cast<size_t>(cols / kSuperBlock) * kQ4KBytes;
    case GUFO_CUDA_Q6_K:
      return cols % kSuperBlock ? 0 : static_cast<size_t>(cols / kSuperBlock) * kQ6KBytes;
    case GUFO_CUDA_Q5_K:
      return cols % kSuperBlock ? 0 : static_cast<size_t>(cols / kSuperBlock) * kQ5KBytes;
    case GUFO_CUDA_Q8_0:
      return cols % kQ8Block ? 0 : static_cast<size_t>(cols / kQ8Block) * kQ8Bytes;
    case GUFO_CUDA_F16:
    case GUFO_CUDA_BF16:
      return static_cast<size_t>(cols) * 2;
    default:
      return 0;
  }
}

size_t DeviceRowBytes(int type, int64_t cols) {
  return type == GUFO_CUDA_Q6_K ? Q6KDeviceRowBytes(cols) : RowBytes(type, cols);
}

namespace {

// One thread per (row, block): moves the 210 bytes of a GGUF Q6_K block to
// their planar places. Runs once per matrix at upload.
__global__ void RepackQ6K(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                          int64_t rows, int blocks, size_t src_row, size_t dst_row) {
  const int64_t item = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (item >= rows * blocks) {
    return;
  }
  const int64_t r = item / blocks;
  const int b = static_cast<int>(item - r * blocks);
  const uint8_t* in = src + r * src_row + static_cast<size_t>(b) * kQ6KBytes;
  const Q6KBlock out = Q6KBlockAt(dst + r * dst_row, blocks, b);
  uint8_t* ql = const_cast<uint8_t*>(out.ql);
  uint8_t* qh = const_cast<uint8_t*>(out.qh);
  uint8_t* sc = reinterpret_cast<uint8_t*>(const_cast<int8_t*>(out.sc));
  uint8_t* d = const_cast<uint8_t*>(out.d);
  // Blocks start on even addresses only: 2-byte moves.
  const uint16_t* in16 = reinterpret_cast<const uint16_t*>(in);
  for (int i = 0; i < 64; ++i) {
    reinterpret_cast<uint16_t*>(ql)[i] = in16[i];
  }
  for (int i = 0; i < 32; ++i) {
    reinterpret_cast<uint16_t*>(qh)[i] = in16[64 + i];
  }
  for (int i = 0; i < 8; ++i) {
    reinterpret_cast<uint16_t*>(sc)[i] = in16[96 + i];
  }
  reinterpret_cast<uint16_t*>(d)[0] = in16[104];
}

}  // namespace

// Copies GGUF Q6_K rows at `raw` (device) into a new planar buffer.
int RepackQ6KRows(gufo_cuda_ctx* ctx, const uint8_t* raw, int64_t rows, int64_t cols,
                  uint8_t** out) {
  const size_t dst_row = Q6KDeviceRowBytes(cols);
  const int blocks = static_cast<int>(cols / kSuperBlock);
  void* dst = nullptr;
  GUFO_CUDA_TRY(cudaMalloc(&dst, dst_row * static_cast<size_t>(rows) + 16));
  cudaError_t e = cudaMemsetAsync(dst, 0, dst_row * static_cast<size_t>(rows) + 16, ctx->stream);
  if (e == cudaSuccess) {
    const int64_t items = rows * blocks;
    const int grid = static_cast<int>((items + 255) / 256);
    RepackQ6K<<<grid, 256, 0, ctx->stream>>>(raw, static_cast<uint8_t*>(dst), rows, blocks,
                                              static_cast<size_t>(blocks) * kQ6KBytes, dst_row);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) {
    e = cudaStreamSynchronize(ctx->stream);
  }
  if (e != cudaSuccess) {
    cudaFree(dst);
    return CudaFail(e, "repack Q6_K");
  }
  *out = static_cast<uint8_t*>(dst);
  return GUFO_CUDA_OK;
}

}  // namespace gufo

int gufo_cuda_ctx::Reserve(float** buffer, size_t* have, size_t want) {
  if (*have >= want) {
    return GUFO_CUDA_OK;
  }
  if (*buffer != nullptr) {
    GUFO_CUDA_TRY(cudaStreamSynchronize(stream));
    GUFO_CUDA_TRY(cudaFree(*buffer));
    *buffer = nullptr;
    *have = 0;
  }
  const size_t grown = want + want / 2;
  GUFO_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(buffer), grown));
  *have = grown;
  return GUFO_CUDA_OK;
}

using gufo::Fail;

extern "C" {

const char* gufo_cuda_last_error(const gufo_cuda_ctx*) {
  return gufo::g_last_error.c_str();
}

int64_t gufo_cuda_launch_count(const gufo_cuda_ctx* ctx) {
  return ctx == nullptr ? 0 : ctx->launches.load();
}

int gufo_cuda_ctx_create(int device, void* stream, gufo_cuda_ctx** out) {
  if (out == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "ctx_create: out is null");
  }
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    return Fail(GUFO_CUDA_RUNTIME,
                std::string("no CUDA device: this backend has no CPU path (") +
                    cudaGetErrorString(e) + ")");
  }
  if (device < 0 || device >= count) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "ctx_create: no such device");
  }
  GUFO_CUDA_TRY(cudaSetDevice(device));
  cudaDeviceProp prop;
  GUFO_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    return Fail(GUFO_CUDA_RUNTIME,
                "device is not sm_100: the kernels are built for sm_100a only");
  }
  auto* ctx = new (std::nothrow) gufo_cuda_ctx();
  if (ctx == nullptr) {
    return Fail(GUFO_CUDA_OUT_OF_MEMORY, "ctx_create: host allocation failed");
  }
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  if (stream != nullptr) {
    ctx->stream = static_cast<cudaStream_t>(stream);
  } else {
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
      delete ctx;
      return gufo::CudaFail(e, "cudaStreamCreate");
    }
    ctx->own_stream = true;
  }
  *out = ctx;
  return GUFO_CUDA_OK;
}

int gufo_cuda_ctx::GrowScratch(uint8_t** block, size_t* have, size_t want, size_t floor, const char* what) {
  if (*have >= want) {
    return GUFO_CUDA_OK;
  }
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capturing) == cudaSuccess && capturing != cudaStreamCaptureStatusNone) {
    return gufo::Fail(GUFO_CUDA_BAD_ARGUMENT,
                      std::string(what) + ": the context's scratch must grow for this product, which a stream "
                                          "capture cannot do; run the product once before capturing");
  }
  const size_t grown = want < floor ? floor : want;
  uint8_t* fresh = nullptr;
  GUFO_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&fresh), grown));
  if (*block != nullptr) {
    retired.push_back(*block);   // a graph captured earlier may still use it
  }
  *block = fresh;
  *have = grown;
  return GUFO_CUDA_OK;
}

int gufo_cuda_ctx_destroy(gufo_cuda_ctx* ctx) {
  if (ctx == nullptr) {
    return GUFO_CUDA_OK;
  }
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  for (auto& kv : ctx->matrices) {
    if (kv.second.owned) {
      cudaFree(const_cast<uint8_t*>(kv.second.data));
    }
  }
  for (auto& kv : ctx->deltanet_layers) {
    cudaFree(kv.second.conv);
    cudaFree(kv.second.ssm_a);
    cudaFree(kv.second.dt_bias);
    cudaFree(kv.second.ssm_norm);
  }
  cudaFree(ctx->stage_x);
  cudaFree(ctx->stage_y);
  cudaFree(ctx->image);
  cudaFree(ctx->tc_scratch);
  for (void* block : ctx->retired) {
    cudaFree(block);
  }
  if (ctx->own_stream) {
    cudaStreamDestroy(ctx->stream);
  }
  delete ctx;
  return GUFO_CUDA_OK;
}

int gufo_cuda_ctx_set_stream(gufo_cuda_ctx* ctx, void* stream) {
  if (ctx == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "set_stream: ctx is null");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (ctx->own_stream) {
    cudaStreamSynchronize(ctx->stream);
    cudaStreamDestroy(ctx->stream);
    ctx->own_stream = false;
  }
  ctx->stream = static_cast<cudaStream_t>(stream);
  return GUFO_CUDA_OK;
}

int gufo_cuda_ctx_set_option(gufo_cuda_ctx* ctx, const char* name, int value) {
  if (ctx == nullptr || name == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "set_option: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (std::strcmp(name, "general_gemv") == 0) {
    ctx->force_general = value != 0;
    return GUFO_CUDA_OK;
  }
  if (std::strcmp(name, "gemv_variant") == 0) {
    ctx->gemv_variant = value;
    return GUFO_CUDA_OK;
  }
  if (std::strcmp(name, "deltanet_early_state") == 0) {
    ctx->early_state = value != 0;
    return GUFO_CUDA_OK;
  }
  if (std::strcmp(name, "tc_gemm") == 0) {
    ctx->tc_gemm = value != 0;
    ctx->tc_gemm_all = value == 2;
    return GUFO_CUDA_OK;
  }
  if (std::strcmp(name, "step_kernel") == 0) {
    ctx->step_kernel = value != 0;
    return GUFO_CUDA_OK;
  }
  if (std::strcmp(name, "step_wait_us") == 0) {
    if (value < 1) {
      return Fail(GUFO_CUDA_BAD_ARGUMENT, "set_option: step_wait_us takes microseconds, at least 1");
    }
    ctx->step_wait_us = value;
    return GUFO_CUDA_OK;
  }
  if (std::strcmp(name, "step_skip_arrival") == 0) {
    ctx->step_skip_arrival = value;
    return GUFO_CUDA_OK;
  }
  if (std::strcmp(name, "reuse_image") == 0) {
    ctx->reuse_image = value != 0;
    return GUFO_CUDA_OK;
  }
  return Fail(GUFO_CUDA_BAD_ARGUMENT, std::string("set_option: unknown option ") + name);
}

int gufo_cuda_ctx_synchronize(gufo_cuda_ctx* ctx) {
  if (ctx == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "synchronize: ctx is null");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  // A bounded wait of the tcgen05 GEMM that ran out leaves its code behind.
  int code = 0;
  const int rc = gufo::TcGemmError(ctx, &code);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  if (code != 0) {
    cudaMemsetAsync(ctx->tc_scratch, 0, sizeof(int), ctx->stream);
    return Fail(GUFO_CUDA_TIMEOUT, "tcgen05 gemm: a wait on a shared-memory barrier ran out (code " +
                                       std::to_string(code) + "); the outputs of that product are invalid");
  }
  return GUFO_CUDA_OK;
}

int gufo_cuda_malloc(gufo_cuda_ctx* ctx, size_t bytes, void** device_ptr) {
  if (ctx == nullptr || device_ptr == nullptr || bytes == 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "malloc: bad argument");
  }
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  GUFO_CUDA_TRY(cudaMalloc(device_ptr, bytes));
  return GUFO_CUDA_OK;
}

int gufo_cuda_free(gufo_cuda_ctx* ctx, void* device_ptr) {
  if (ctx == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "free: ctx is null");
  }
  if (device_ptr != nullptr) {
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    GUFO_CUDA_TRY(cudaFree(device_ptr));
  }
  return GUFO_CUDA_OK;
}

int gufo_cuda_upload(gufo_cuda_ctx* ctx, void* device_dst, const void* host_src,
                     size_t bytes) {
  if (ctx == nullptr || device_dst == nullptr || host_src == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "upload: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaMemcpyAsync(device_dst, host_src, bytes,
                                cudaMemcpyHostToDevice, ctx->stream));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  return GUFO_CUDA_OK;
}

int gufo_cuda_download(gufo_cuda_ctx* ctx, void* host_dst,
                       const void* device_src, size_t bytes) {
  if (ctx == nullptr || host_dst == nullptr || device_src == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "download: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaMemcpyAsync(host_dst, device_src, bytes,
                                cudaMemcpyDeviceToHost, ctx->stream));
  GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  return GUFO_CUDA_OK;
}

int gufo_cuda_memset_zero(gufo_cuda_ctx* ctx, void* device_ptr, size_t bytes) {
  if (ctx == nullptr || device_ptr == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "memset_zero: null pointer");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaMemsetAsync(device_ptr, 0, bytes, ctx->stream));
  return GUFO_CUDA_OK;
}

static int AddMatrix(gufo_cuda_ctx* ctx, int type, const uint8_t* data,
                     int64_t rows, int64_t cols, bool owned,
                     gufo_cuda_matrix* out) {
  gufo::Matrix m;
  m.type = type;
  m.data = data;
  m.rows = rows;
  m.cols = cols;
  m.row_bytes = gufo::DeviceRowBytes(type, cols);
  m.owned = owned;
  const int64_t id = ctx->next_id++;
  ctx->matrices.emplace(id, m);
  *out = id;
  return GUFO_CUDA_OK;
}

static int CheckMatrixArgs(const gufo_cuda_ctx* ctx, int type, const void* bytes,
                           int64_t rows, int64_t cols,
                           const gufo_cuda_matrix* out) {
  if (ctx == nullptr || bytes == nullptr || out == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matrix: null pointer");
  }
  if (type != GUFO_CUDA_F32 && type != GUFO_CUDA_Q4_K && type != GUFO_CUDA_Q6_K && type != GUFO_CUDA_Q5_K &&
      type != GUFO_CUDA_Q8_0 && type != GUFO_CUDA_F16 && type != GUFO_CUDA_BF16) {
    return Fail(GUFO_CUDA_UNSUPPORTED_TYPE,
                "matrix: ggml type " + std::to_string(type) +
                    " is not run by this backend (Q4_K, Q5_K, Q6_K, Q8_0, F32, F16, BF16)");
  }
  if (rows <= 0 || cols <= 0) {
    return Fail(GUFO_CUDA_SHAPE, "matrix: rows and cols must be positive");
  }
  if (gufo::RowBytes(type, cols) == 0) {
    return Fail(GUFO_CUDA_SHAPE, "matrix: row is not a whole number of blocks");
  }
  if (type == GUFO_CUDA_F32 && cols % 4 != 0) {
    return Fail(GUFO_CUDA_SHAPE, "matrix: F32 rows must be a multiple of 4 wide");
  }
  return GUFO_CUDA_OK;
}

int gufo_cuda_matrix_upload(gufo_cuda_ctx* ctx, int ggml_type,
                            const void* host_bytes, int64_t rows, int64_t cols,
                            gufo_cuda_matrix* out) {
  int rc = CheckMatrixArgs(ctx, ggml_type, host_bytes, rows, cols, out);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
  const size_t bytes = gufo::RowBytes(ggml_type, cols) * static_cast<size_t>(rows);
  // 16 spare bytes: kernels may read whole 16-byte vectors up to the end.
  void* dev = nullptr;
  GUFO_CUDA_TRY(cudaMalloc(&dev, bytes + 16));
  cudaError_t e = cudaMemcpyAsync(dev, host_bytes, bytes, cudaMemcpyHostToDevice,
                                  ctx->stream);
  if (e == cudaSuccess) {
    e = cudaStreamSynchronize(ctx->stream);
  }
  if (e != cudaSuccess) {
    cudaFree(dev);
    return gufo::CudaFail(e, "matrix_upload copy");
  }
  if (ggml_type == GUFO_CUDA_Q6_K) {
    uint8_t* planar = nullptr;
    rc = gufo::RepackQ6KRows(ctx, static_cast<const uint8_t*>(dev), rows, cols, &planar);
    cudaFree(dev);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
    dev = planar;
  }
  return AddMatrix(ctx, ggml_type, static_cast<const uint8_t*>(dev), rows, cols,
                   true, out);
}

int gufo_cuda_matrix_from_device(gufo_cuda_ctx* ctx, int ggml_type,
                                 const void* device_bytes, int64_t rows,
                                 int64_t cols, gufo_cuda_matrix* out) {
  int rc = CheckMatrixArgs(ctx, ggml_type, device_bytes, rows, cols, out);
  if (rc != GUFO_CUDA_OK) {
    return rc;
  }
  if (reinterpret_cast<uintptr_t>(device_bytes) % 16 != 0) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT,
                "matrix_from_device: bytes must be 16-byte aligned");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  if (ggml_type == GUFO_CUDA_Q6_K) {
    // Q6_K is rearranged into its planar device form: a copy, owned here.
    GUFO_CUDA_TRY(cudaSetDevice(ctx->device));
    uint8_t* planar = nullptr;
    rc = gufo::RepackQ6KRows(ctx, static_cast<const uint8_t*>(device_bytes), rows, cols, &planar);
    if (rc != GUFO_CUDA_OK) {
      return rc;
    }
    return AddMatrix(ctx, ggml_type, planar, rows, cols, true, out);
  }
  return AddMatrix(ctx, ggml_type, static_cast<const uint8_t*>(device_bytes), rows,
                   cols, false, out);
}

int gufo_cuda_matrix_free(gufo_cuda_ctx* ctx, gufo_cuda_matrix matrix) {
  if (ctx == nullptr) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matrix_free: ctx is null");
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  auto it = ctx->matrices.find(matrix);
  if (it == ctx->matrices.end()) {
    return Fail(GUFO_CUDA_BAD_ARGUMENT, "matrix_free: unknown handle");
  }
  if (it->second.owned) {
    GUFO_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    GUFO_CUDA_TRY(cudaFree(const_cast<uint8_t*>(it->second.data)));
  }
  ctx->matrices.erase(it);
  return GUFO_CUDA_OK;
}

}  // extern "C"
