// Gated-FFN forward for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run the FFN: code
// that runs inside a memory-pool or arena owner which forbids side allocations, real-time serving
// loops where an allocation may block on the driver or fragment a carefully packed device, and
// embedders that hand this library a fixed device budget up front.  The regular entry point,
// sfb200_ffn_forward, needs an M x I scratch tensor for the hidden activations from its caller, and
// the host-buffer entry point grows library-owned staging buffers on demand.  This variant keeps
// that scratch in a fixed array that is part of the library image instead, so nothing is allocated
// or freed, here or in anything it calls.
//
// Cost and limits: every GPU that loads the library carries the array (kScratchBytes) until the
// process exits; problems whose hidden tensor (M * I * 2 bytes) does not fit are refused with
// SFB200_ERROR_SCRATCH_TOO_SMALL.  The array is shared by every call on a device and keeps the last
// call's contents: calls that overlap on the GPU (different streams, or threads) race on it, so
// callers serialise them.  Nothing in it has to start at zero: the gate|up kernel writes every
// element of the M x I region before the down kernel reads it.
//
// The first call on each device looks up the array's device address (and sets kernel attributes);
// make that call before starting any stream capture.  "Allocates nothing" is a statement about this
// library's own calls: the CUDA runtime may still load a kernel's module the first time that kernel
// is launched on a device, which is one more reason to make the first call during start-up.
//
// Device-side failures (a bounded wait that ran out) of this entry point are recorded in a status
// word that is also part of the library image; sfb200_noalloc_device_status reads and clears it
// without allocating, and sfb200_device_status includes it.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

#include "../../include/sparseflow_b200.h"
#include "device_state.h"
#include "kernels.h"

namespace sfb200 {
namespace {

constexpr size_t kScratchBytes = SFB200_NOALLOC_SCRATCH_BYTES;

// In host code these names are only stand-ins for the symbols: the device addresses come from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_hidden_scratch[kScratchBytes];
static __device__ __align__(256) int g_status_word[64];

struct NoAllocDevice {
  std::atomic<bool> ready{false};
  void* scratch = nullptr;
  int* status = nullptr;
  int num_sms = 0;
};
NoAllocDevice g_dev[kMaxDevices];
std::mutex g_mu;

// Once per device, with that device current.
int setup_current_device(NoAllocDevice** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return kErrCuda;
  }
  NoAllocDevice* d = &g_dev[dev];
  if (!d->ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!d->ready.load(std::memory_order_relaxed)) {
      int major = 0, sms = 0;
      if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
          cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();
        return kErrCuda;
      }
      if (major != 10) return kErrNotSupported;
      void* sp = nullptr;
      void* st = nullptr;
      if (cudaGetSymbolAddress(&sp, g_hidden_scratch) != cudaSuccess ||
          cudaGetSymbolAddress(&st, g_status_word) != cudaSuccess) {
        cudaGetLastError();
        return kErrCuda;
      }
      d->scratch = sp;
      d->status = static_cast<int*>(st);
      d->num_sms = sms;
      d->ready.store(true, std::memory_order_release);
    }
  }
  *out = d;
  return kOk;
}

}  // namespace

// Device address of that status word on the current device (performs the per-device set-up if needed);
// nullptr when the device is unusable.  Used by the bounded-wait probe to exercise this word's read path.
int* noalloc_status_word() {
  NoAllocDevice* d = nullptr;
  return setup_current_device(&d) == kOk ? d->status : nullptr;
}

// Status word of the allocation-free entry point on the current device: synchronises, reads and
// clears it.  *word = 0 and kOk when that entry point has not run on this device.
int noalloc_take_status(int* word) {
  *word = 0;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return kErrCuda;
  }
  NoAllocDevice* d = &g_dev[dev];
  if (!d->ready.load(std::memory_order_acquire)) return kOk;
  if (cudaDeviceSynchronize() != cudaSuccess) return kErrCuda;
  int w = 0;
  if (cudaMemcpy(&w, d->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return kErrCuda;
  if (w != 0 && cudaMemset(d->status, 0, sizeof(int)) != cudaSuccess) return kErrCuda;
  *word = w;
  return kOk;
}

}  // namespace sfb200

using namespace sfb200;

extern "C" int sfb200_noalloc_device_status(int* status_word) {
  int w = 0;
  const int rc = noalloc_take_status(&w);
  if (status_word) *status_word = w;
  if (rc != kOk) return rc;
  return w == 0 ? kOk : kErrDevice;
}

extern "C" int sfb200_ffn_forward_noalloc(const sfb200_ffn_weights* w, const void* x, int ldx, void* out,
                                          int ldo, int M, void* stream) {
  if (!w || !x || !out || M <= 0 || w->H <= 0 || w->I <= 0) return kErrInvalid;
  if (!w->gu_values || !w->gu_meta || !w->down_values || !w->down_meta) return kErrInvalid;
  if (w->dtype != kF16 && w->dtype != kBF16) return kErrInvalid;
  const size_t need = static_cast<size_t>(M) * static_cast<size_t>(w->I) * 2;
  if (need > kScratchBytes) return SFB200_ERROR_SCRATCH_TOO_SMALL;
  NoAllocDevice* d = nullptr;
  const int rc0 = setup_current_device(&d);
  if (rc0 != kOk) return rc0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  SparseGemmArgs a{};
  a.x = x;
  a.values = w->gu_values;
  a.meta = w->gu_meta;
  a.y = d->scratch;                 // hidden[M, I] lives in the static array
  a.status = d->status;
  a.m_tok = M;
  a.n_out = 2 * w->I;
  a.K = w->H;
  a.ldx = ldx;
  a.ldy = w->I;
  a.fmt = w->dtype;
  a.epi = kEpiSwiGLU;
  a.act = kActNone;
  a.num_sms = d->num_sms;
  int rc = launch_sparse_gemm(a, st);
  if (rc != kOk) return rc;

  SparseGemmArgs b{};
  b.x = d->scratch;
  b.values = w->down_values;
  b.meta = w->down_meta;
  b.y = out;
  b.bias = w->down_bias;
  b.status = d->status;
  b.m_tok = M;
  b.n_out = w->H;
  b.K = w->I;
  b.ldx = w->I;
  b.ldy = ldo;
  b.fmt = w->dtype;
  b.epi = kEpiStore;
  b.act = kActNone;
  b.num_sms = d->num_sms;
  return launch_sparse_gemm(b, st);
}
