// "Stable C ABI v1" of the reference (experiments/old_structure/include/sparseflow/c_api.h:38-200),
// with the compute entry points that upstream leaves as NOT_SUPPORTED stubs
// (src/runtime/context.cpp:248-300) implemented on the sm_100a kernels.
//
// Conventions kept from upstream: every call returns a SparseFlowStatus; the last error text is
// thread-local (context.cpp:14,92-94); NULL out-pointer => INVALID_ARGUMENT, NULL handle =>
// INVALID_HANDLE, bad device id => INVALID_ARGUMENT (context.cpp:127-146); ABI compatibility is
// "same major" (context.cpp:108-111); data pointers are device pointers; nothing synchronises
// except validate (host result) and benchmark.
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/sparseflow_b200.h"
#include "device_state.h"
#include "kernels.h"

using namespace sfb200;

namespace {

thread_local std::string t_last_error;

constexpr uint32_t kCtxMagic = 0x5F43B200u;
constexpr uint32_t kKernelMagic = 0x5F4BB200u;

SparseFlowStatus fail(SparseFlowStatus s, const std::string& msg) {
  t_last_error = msg;
  return s;
}

SparseFlowStatus from_err(int e, const char* what) {
  switch (e) {
    case kOk: return SPARSEFLOW_SUCCESS;
    case kErrInvalid: return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, std::string(what) + ": invalid argument");
    case kErrOutOfMemory: return fail(SPARSEFLOW_ERROR_OUT_OF_MEMORY, std::string(what) + ": out of device memory");
    case kErrNotSupported: return fail(SPARSEFLOW_ERROR_NOT_SUPPORTED, std::string(what) + ": needs an sm_100 device");
    default: return fail(SPARSEFLOW_ERROR_CUDA_ERROR, std::string(what) + ": CUDA error");
  }
}

int map_dtype(SparseFlowDataType dt) {
  if (dt == SPARSEFLOW_DTYPE_FP16) return kF16;
  if (dt == SPARSEFLOW_DTYPE_BF16) return kBF16;
  return -1;
}

class DeviceGuard {
 public:
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev_);
    if (prev_ != dev) cudaSetDevice(dev);
  }
  ~DeviceGuard() { cudaSetDevice(prev_); }
 private:
  int prev_ = 0;
};

}  // namespace

struct SparseFlowContext_ {
  uint32_t magic;
  int device_id;
  int cc;
  int sm_count;
  size_t total_mem;
};

struct SparseFlowKernel_ {
  uint32_t magic;
  SparseFlowContext_* ctx;
  SparseFlowKernelConfig config;
};

static bool ctx_ok(SparseFlowContext c) { return c && c->magic == kCtxMagic; }
static bool kernel_ok(SparseFlowKernel k) { return k && k->magic == kKernelMagic && ctx_ok(k->ctx); }

extern "C" {

const char* sparseflow_get_error_string(SparseFlowStatus status) {
  switch (status) {
    case SPARSEFLOW_SUCCESS: return "Success";
    case SPARSEFLOW_ERROR_INVALID_ARGUMENT: return "Invalid argument";
    case SPARSEFLOW_ERROR_OUT_OF_MEMORY: return "Out of memory";
    case SPARSEFLOW_ERROR_CUDA_ERROR: return "CUDA error";
    case SPARSEFLOW_ERROR_NOT_SUPPORTED: return "Operation not supported";
    case SPARSEFLOW_ERROR_INVALID_HANDLE: return "Invalid handle";
    case SPARSEFLOW_ERROR_COMPILATION_FAILED: return "Kernel compilation failed";
    case SPARSEFLOW_ERROR_ABI_MISMATCH: return "ABI version mismatch";
    default: return "Unknown error";
  }
}

const char* sparseflow_get_last_error(void) { return t_last_error.c_str(); }

SparseFlowVersion sparseflow_get_version(void) {
  SparseFlowVersion v = {SPARSEFLOW_ABI_VERSION_MAJOR, SPARSEFLOW_ABI_VERSION_MINOR,
                         SPARSEFLOW_ABI_VERSION_PATCH};
  return v;
}

int sparseflow_is_abi_compatible(int major, int /*minor*/) {
  return major == SPARSEFLOW_ABI_VERSION_MAJOR ? 1 : 0;
}

SparseFlowStatus sparseflow_create_context(SparseFlowContext* ctx, int device_id) {
  if (!ctx) return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "ctx is NULL");
  *ctx = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return fail(SPARSEFLOW_ERROR_CUDA_ERROR, "cudaGetDeviceCount failed (no CUDA device?)");
  }
  if (device_id < 0 || device_id >= count)
    return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "Invalid device ID: " + std::to_string(device_id));
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device_id) != cudaSuccess) {
    cudaGetLastError();
    return fail(SPARSEFLOW_ERROR_CUDA_ERROR, "cudaGetDeviceProperties failed");
  }
  SparseFlowContext_* c = new (std::nothrow) SparseFlowContext_;
  if (!c) return fail(SPARSEFLOW_ERROR_OUT_OF_MEMORY, "host allocation failed");
  c->magic = kCtxMagic;
  c->device_id = device_id;
  c->cc = prop.major * 10 + prop.minor;
  c->sm_count = prop.multiProcessorCount;
  c->total_mem = prop.totalGlobalMem;
  *ctx = c;
  return SPARSEFLOW_SUCCESS;
}

SparseFlowStatus sparseflow_destroy_context(SparseFlowContext ctx) {
  if (!ctx_ok(ctx)) return fail(SPARSEFLOW_ERROR_INVALID_HANDLE, "invalid context handle");
  ctx->magic = 0;
  delete ctx;
  return SPARSEFLOW_SUCCESS;
}

SparseFlowStatus sparseflow_get_device_info(SparseFlowContext ctx, int* compute_capability,
                                            int* sm_count, size_t* total_memory) {
  if (!ctx_ok(ctx)) return fail(SPARSEFLOW_ERROR_INVALID_HANDLE, "invalid context handle");
  if (compute_capability) *compute_capability = ctx->cc;
  if (sm_count) *sm_count = ctx->sm_count;
  if (total_memory) *total_memory = ctx->total_mem;
  return SPARSEFLOW_SUCCESS;
}

SparseFlowStatus sparseflow_compile_kernel(SparseFlowContext ctx, SparseFlowKernel* kernel,
                                           const SparseFlowKernelConfig* config) {
  if (!ctx_ok(ctx)) return fail(SPARSEFLOW_ERROR_INVALID_HANDLE, "invalid context handle");
  if (!kernel || !config) return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "kernel or config is NULL");
  *kernel = nullptr;
  if (config->epilogue.kind < SPARSEFLOW_EPILOGUE_NONE || config->epilogue.kind > SPARSEFLOW_EPILOGUE_BIAS_SILU)
    return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "unknown epilogue kind");
  const bool wants_bias = config->epilogue.kind >= SPARSEFLOW_EPILOGUE_BIAS;
  if (wants_bias && config->epilogue.params == nullptr)
    return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "BIAS epilogue needs params = device bias pointer");
  const int tn = config->tile_n;
  if (!(tn == 0 || tn == 32 || tn == 64 || tn == 128 || tn == 192 || tn == 256))
    return fail(SPARSEFLOW_ERROR_COMPILATION_FAILED, "tile_n must be 0, 32, 64, 128, 192 or 256");
  if (ctx->cc / 10 != 10)
    return fail(SPARSEFLOW_ERROR_NOT_SUPPORTED, "kernels are built for sm_100a only");
  SparseFlowKernel_* k = new (std::nothrow) SparseFlowKernel_;
  if (!k) return fail(SPARSEFLOW_ERROR_OUT_OF_MEMORY, "host allocation failed");
  k->magic = kKernelMagic;
  k->ctx = ctx;
  k->config = *config;
  *kernel = k;
  return SPARSEFLOW_SUCCESS;
}

SparseFlowStatus sparseflow_destroy_kernel(SparseFlowKernel kernel) {
  if (!kernel || kernel->magic != kKernelMagic)
    return fail(SPARSEFLOW_ERROR_INVALID_HANDLE, "invalid kernel handle");
  kernel->magic = 0;
  delete kernel;
  return SPARSEFLOW_SUCCESS;
}

size_t sparseflow_compressed_meta_offset(int N, int K) {
  const size_t v = values_bytes(N, K);
  return (v + 255) & ~static_cast<size_t>(255);
}

SparseFlowStatus sparseflow_sparse_gemm(SparseFlowKernel kernel, const void* A, const void* Bc, void* C,
                                        int M, int N, int K, SparseFlowDataType dtype, void* stream) {
  if (!kernel_ok(kernel)) return fail(SPARSEFLOW_ERROR_INVALID_HANDLE, "invalid kernel handle");
  if (!A || !Bc || !C) return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "NULL matrix pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "non-positive dimension");
  const int fmt = map_dtype(dtype);
  if (fmt < 0) return fail(SPARSEFLOW_ERROR_NOT_SUPPORTED, "only FP16 and BF16 have a sparse kernel");
  DeviceGuard g(kernel->ctx->device_id);
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return from_err(err, "sparseflow_sparse_gemm");
  const SparseFlowEpilogue ek = kernel->config.epilogue.kind;
  int act = kActNone;
  if (ek == SPARSEFLOW_EPILOGUE_RELU || ek == SPARSEFLOW_EPILOGUE_BIAS_RELU) act = kActRelu;
  if (ek == SPARSEFLOW_EPILOGUE_SILU || ek == SPARSEFLOW_EPILOGUE_BIAS_SILU) act = kActSilu;
  if (ek == SPARSEFLOW_EPILOGUE_GELU) act = kActGelu;
  SparseGemmArgs a{};
  a.x = A;
  a.values = Bc;
  a.meta = static_cast<const uint8_t*>(Bc) + sparseflow_compressed_meta_offset(N, K);
  a.y = C;
  a.bias = ek >= SPARSEFLOW_EPILOGUE_BIAS ? kernel->config.epilogue.params : nullptr;
  a.status = s->status;
  a.m_tok = M;
  a.n_out = N;
  a.K = K;
  a.ldx = K;
  a.ldy = N;
  a.fmt = fmt;
  a.epi = kEpiStore;
  a.act = act;
  a.num_sms = s->num_sms;
  a.force_bn = kernel->config.tile_n;
  return from_err(launch_sparse_gemm(a, static_cast<cudaStream_t>(stream)), "sparseflow_sparse_gemm");
}

SparseFlowStatus sparseflow_compress_2_4(SparseFlowContext ctx, const void* dense, void* compressed,
                                         void* metadata, int M, int N, SparseFlowDataType dtype) {
  if (!ctx_ok(ctx)) return fail(SPARSEFLOW_ERROR_INVALID_HANDLE, "invalid context handle");
  if (!dense || !compressed || !metadata) return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "NULL pointer");
  if (M <= 0 || N <= 0 || N % 16 != 0)
    return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "need M > 0 and N a positive multiple of 16");
  const int fmt = map_dtype(dtype);
  if (fmt < 0) return fail(SPARSEFLOW_ERROR_NOT_SUPPORTED, "only FP16 and BF16 are supported");
  DeviceGuard g(ctx->device_id);
  int err = kOk;
  if (!device_state(&err)) return from_err(err, "sparseflow_compress_2_4");
  PruneArgs a{};
  a.dense = dense;
  a.rows = M;
  a.K = N;
  a.ld = N;
  a.fmt = fmt;
  a.tie = kTieHigh;
  a.values = compressed;
  a.meta = metadata;
  return from_err(launch_prune_compress(a, nullptr), "sparseflow_compress_2_4");
}

SparseFlowStatus sparseflow_validate_2_4(const void* tensor, int M, int N, SparseFlowDataType dtype,
                                         int* is_valid) {
  if (!tensor || !is_valid) return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "NULL pointer");
  if (M <= 0 || N <= 0 || N % 4 != 0)
    return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "need M > 0 and N a positive multiple of 4");
  if (map_dtype(dtype) < 0) return fail(SPARSEFLOW_ERROR_NOT_SUPPORTED, "only FP16 and BF16 are supported");
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return from_err(err, "sparseflow_validate_2_4");
  int* flag = s->status + 8;  // scratch word inside the status allocation
  const int one = 1;
  if (cudaMemcpy(flag, &one, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess)
    return fail(SPARSEFLOW_ERROR_CUDA_ERROR, "cudaMemcpy failed");
  const int rc = launch_validate_24(tensor, M, N, N, flag, nullptr);
  if (rc != kOk) return from_err(rc, "sparseflow_validate_2_4");
  int out = 0;
  if (cudaMemcpy(&out, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
    return fail(SPARSEFLOW_ERROR_CUDA_ERROR, "cudaMemcpy failed");
  *is_valid = out;
  return SPARSEFLOW_SUCCESS;
}

SparseFlowStatus sparseflow_benchmark_kernel(SparseFlowKernel kernel, int M, int N, int K,
                                             int num_iterations, SparseFlowBenchmarkResult* result) {
  if (!kernel_ok(kernel)) return fail(SPARSEFLOW_ERROR_INVALID_HANDLE, "invalid kernel handle");
  if (!result) return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "result is NULL");
  if (M <= 0 || N <= 0 || K <= 0 || K % 64 != 0 || N % 8 != 0 || num_iterations <= 0)
    return fail(SPARSEFLOW_ERROR_INVALID_ARGUMENT, "need M, N > 0, N % 8 == 0, K % 64 == 0, iterations > 0");
  DeviceGuard g(kernel->ctx->device_id);
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return from_err(err, "sparseflow_benchmark_kernel");
  const size_t wb = static_cast<size_t>(N) * K * 2, xb = static_cast<size_t>(M) * K * 2,
               yb = static_cast<size_t>(M) * N * 2;
  void *w = nullptr, *x = nullptr, *y = nullptr, *blk = nullptr;
  const size_t moff = sparseflow_compressed_meta_offset(N, K);
  auto free_all = [&] {
    for (void* p : {w, x, y, blk})
      if (p) cudaFree(p);
  };
  if (cudaMalloc(&w, wb) || cudaMalloc(&x, xb) || cudaMalloc(&y, yb) ||
      cudaMalloc(&blk, moff + meta_bytes(N, K))) {
    cudaGetLastError();
    free_all();
    return fail(SPARSEFLOW_ERROR_OUT_OF_MEMORY, "benchmark buffers do not fit");
  }
  {
    std::vector<uint16_t> hw(static_cast<size_t>(N) * K), hx(static_cast<size_t>(M) * K);
    uint32_t st = 12345u;
    auto rnd = [&] { st = st * 1664525u + 1013904223u; return st; };
    for (auto& v : hw) v = static_cast<uint16_t>(0x2000 + (rnd() >> 20)) | static_cast<uint16_t>((rnd() >> 31) << 15);
    for (auto& v : hx) v = static_cast<uint16_t>(0x3800 + (rnd() >> 22)) | static_cast<uint16_t>((rnd() >> 31) << 15);
    cudaMemcpy(w, hw.data(), wb, cudaMemcpyHostToDevice);
    cudaMemcpy(x, hx.data(), xb, cudaMemcpyHostToDevice);
  }
  SparseFlowStatus rc = sparseflow_compress_2_4(kernel->ctx, w, blk, static_cast<uint8_t*>(blk) + moff, N, K,
                                                SPARSEFLOW_DTYPE_FP16);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (rc == SPARSEFLOW_SUCCESS && (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess))
    rc = fail(SPARSEFLOW_ERROR_CUDA_ERROR, "cudaEventCreate failed");
  if (rc == SPARSEFLOW_SUCCESS) {
    for (int i = 0; i < 3 && rc == SPARSEFLOW_SUCCESS; ++i)
      rc = sparseflow_sparse_gemm(kernel, x, blk, y, M, N, K, SPARSEFLOW_DTYPE_FP16, nullptr);
    cudaEventRecord(e0, nullptr);
    for (int i = 0; i < num_iterations && rc == SPARSEFLOW_SUCCESS; ++i)
      rc = sparseflow_sparse_gemm(kernel, x, blk, y, M, N, K, SPARSEFLOW_DTYPE_FP16, nullptr);
    cudaEventRecord(e1, nullptr);
    if (cudaEventSynchronize(e1) != cudaSuccess) rc = fail(SPARSEFLOW_ERROR_CUDA_ERROR, "benchmark launch failed");
  }
  if (rc == SPARSEFLOW_SUCCESS) {
    int word = 0;
    cudaMemcpy(&word, s->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (word != 0) {
      cudaMemset(s->status, 0, sizeof(int));
      rc = fail(SPARSEFLOW_ERROR_CUDA_ERROR, "device-side failure, status word " + std::to_string(word));
    }
  }
  if (rc == SPARSEFLOW_SUCCESS) {
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    const double t = static_cast<double>(ms) / num_iterations;
    const double flops = 2.0 * M * N * K;
    result->elapsed_ms = t;
    result->tflops_effective = flops / (t * 1e9);
    result->tflops_real = 0.5 * flops / (t * 1e9);
    const double bytes = static_cast<double>(xb) + values_bytes(N, K) + static_cast<double>(N) * K / 8 + yb;
    result->bandwidth_gb_s = bytes / (t * 1e6);
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  free_all();
  return rc;
}

}  // extern "C"
