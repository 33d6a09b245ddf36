// C-ABI entry points of the hot path (group 1 of include/sparseflow_b200.h).
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include <nvtx3/nvToolsExt.h>

#include "../../include/sparseflow_b200.h"
#include "device_state.h"
#include "kernels.h"

using namespace sfb200;

namespace {
// NVTX range around the host side of a launch sequence (prune, gate|up GEMM, down GEMM, exchange):
// shows up in a timeline tool when one is attached, costs a pointer test otherwise.
struct Range {
  explicit Range(const char* name) { nvtxRangePushA(name); }
  ~Range() { nvtxRangePop(); }
};
}  // namespace

namespace sfb200 {

static DeviceState g_states[kMaxDevices];
static std::mutex g_state_mu;

DeviceState* device_state(int* err) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    if (err) *err = kErrCuda;
    cudaGetLastError();
    return nullptr;
  }
  DeviceState* s = &g_states[dev];
  if (s->ready.load(std::memory_order_acquire)) return s;
  std::lock_guard<std::mutex> lk(g_state_mu);
  if (s->ready.load(std::memory_order_relaxed)) return s;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
    if (err) *err = kErrCuda;
    cudaGetLastError();
    return nullptr;
  }
  s->cc = prop.major * 10 + prop.minor;
  s->num_sms = prop.multiProcessorCount;
  s->total_mem = prop.totalGlobalMem;
  if (prop.major != 10) {  // kernels are sm_100a only
    if (err) *err = kErrNotSupported;
    return nullptr;
  }
  if (cudaMalloc(&s->status, 256) != cudaSuccess || cudaMemset(s->status, 0, 256) != cudaSuccess) {
    if (err) *err = kErrOutOfMemory;
    cudaGetLastError();
    return nullptr;
  }
  s->ready.store(true, std::memory_order_release);
  return s;
}

}  // namespace sfb200

// Token-chunk plan of the host-buffer pipeline; returns the number of chunks (<= kMaxChunks),
// sizes in out[], multiples of 8 except the last.  main_rows / tail_rows <= 0 select the defaults.
int plan_host_chunks(int M, int main_rows, int tail_rows, int* out) {
  constexpr int kMax = DeviceState::kMaxChunks;
  if (main_rows <= 0) main_rows = 1024;
  if (tail_rows <= 0) tail_rows = 1024;  // measured on B200 + PCIe 5: halving the tail did not pay (0.976 vs 0.995 ms at 4096 tokens)
  if (tail_rows > main_rows) tail_rows = main_rows;
  // at most kMax - 3 main chunks, so the halving tail always has room
  const int min_main = (M + (kMax - 3) - 1) / (kMax - 3);
  if (main_rows < min_main) main_rows = min_main;
  main_rows = (main_rows + 7) & ~7;
  int n = 0, rem = M;
  while (rem > main_rows && n < kMax - 3) {
    out[n++] = main_rows;
    rem -= main_rows;
  }
  while (rem > tail_rows && n < kMax - 1) {
    int half = ((rem + 1) / 2 + 7) & ~7;
    if (half >= rem) break;
    out[n++] = half;
    rem -= half;
  }
  if (rem > 0) out[n++] = rem;
  return n;
}

extern "C" {

const char* sfb200_status_string(int status) {
  switch (status) {
    case SFB200_SUCCESS: return "success";
    case SFB200_ERROR_INVALID_ARGUMENT: return "invalid argument";
    case SFB200_ERROR_OUT_OF_MEMORY: return "out of device memory";
    case SFB200_ERROR_CUDA: return "CUDA error (no usable device, or a launch failed)";
    case SFB200_ERROR_NOT_SUPPORTED: return "not supported (device is not sm_100, or a layout version this library does not read)";
    case SFB200_ERROR_TENSOR_MAP: return "TMA tensor map could not be encoded";
    case SFB200_ERROR_DEVICE: return "device-side failure (bounded wait ran out)";
    case SFB200_ERROR_SCRATCH_TOO_SMALL:
      return "hidden tensor (M * I * 2 bytes) exceeds the static scratch of sfb200_ffn_forward_noalloc";
    default: return "unknown status";
  }
}

int sfb200_version(void) { return 100; }

size_t sfb200_values_bytes(int rows, int K) { return values_bytes(rows, K); }
size_t sfb200_meta_bytes(int rows, int K) { return meta_bytes(rows, K); }

int sfb200_device_status(int* status_word) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  if (cudaDeviceSynchronize() != cudaSuccess) return kErrCuda;
  int w = 0;
  if (cudaMemcpy(&w, s->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return kErrCuda;
  if (w != 0) cudaMemset(s->status, 0, sizeof(int));
  // the allocation-free FFN entry point keeps its own word (in the library image); fold it in
  int wn = 0;
  if (noalloc_take_status(&wn) != kOk) return kErrCuda;
  if (w == 0) w = wn;
  if (status_word) *status_word = w;
  return w == 0 ? kOk : kErrDevice;
}

int sfb200_prune_compress_24(const void* dense, int rows, int K, int ld, int dtype, int tie,
                             void* values, void* meta, void* ref_codes, void* pruned, void* stream) {
  int err = kOk;
  if (!device_state(&err)) return err;
  Range r("sfb200.prune_compress");
  PruneArgs a{};
  a.dense = dense;
  a.rows = rows;
  a.K = K;
  a.ld = ld;
  a.fmt = dtype;
  a.tie = tie;
  a.values = values;
  a.meta = meta;
  a.ref_codes = ref_codes;
  a.pruned = pruned;
  return launch_prune_compress(a, static_cast<cudaStream_t>(stream));
}

int sfb200_prune_compress_gate_up(const void* gate, const void* up, int I, int K, int ld, int dtype,
                                  int tie, void* values, void* meta, void* stream) {
  int err = kOk;
  if (!device_state(&err)) return err;
  if (gate == nullptr || up == nullptr || I % 16 != 0) return kErrInvalid;
  Range r("sfb200.prune_compress_gate_up");
  PruneArgs a{};
  a.dense = gate;
  a.dense2 = up;
  a.rows = I;
  a.K = K;
  a.ld = ld;
  a.fmt = dtype;
  a.tie = tie;
  a.interleave = 16;
  a.values = values;
  a.meta = meta;
  return launch_prune_compress(a, static_cast<cudaStream_t>(stream));
}

int sfb200_validate_24(const void* w, int rows, int K, int ld, int* is_valid_dev, void* stream) {
  int err = kOk;
  if (!device_state(&err)) return err;
  if (w == nullptr || is_valid_dev == nullptr) return kErrInvalid;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int one = 1;
  if (cudaMemcpyAsync(is_valid_dev, &one, sizeof(int), cudaMemcpyHostToDevice, st) != cudaSuccess)
    return kErrCuda;
  return launch_validate_24(w, rows, K, ld, is_valid_dev, st);
}

int sfb200_decompress_24(const void* values, const void* meta, int rows, int K, void* dense, int ld,
                         void* stream) {
  int err = kOk;
  if (!device_state(&err)) return err;
  if (!values || !meta || !dense) return kErrInvalid;
  return launch_decompress(values, meta, rows, K, dense, ld, static_cast<cudaStream_t>(stream));
}

static int run_gemm(DeviceState* s, const void* x, int ldx, const void* values, const void* meta,
                    void* y, int ldy, int M, int N, int K, int dtype, const void* bias, int act,
                    int epi, int force_bn, cudaStream_t st) {
  if (!x || !values || !meta || !y) return kErrInvalid;
  if (dtype != kF16 && dtype != kBF16) return kErrInvalid;
  SparseGemmArgs a{};
  a.x = x;
  a.values = values;
  a.meta = meta;
  a.y = y;
  a.bias = bias;
  a.status = s->status;
  a.m_tok = M;
  a.n_out = N;
  a.K = K;
  a.ldx = ldx;
  a.ldy = ldy;
  a.fmt = dtype;
  a.epi = epi;
  a.act = act;
  a.num_sms = s->num_sms;
  a.force_bn = force_bn ? force_bn : s->force_bn;
  return launch_sparse_gemm(a, st);
}

int sfb200_sparse_gemm(const void* x, int ldx, const void* values, const void* meta, void* y,
                       int ldy, int M, int N, int K, int dtype, const void* bias, int act,
                       void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  Range r("sfb200.sparse_gemm");
  return run_gemm(s, x, ldx, values, meta, y, ldy, M, N, K, dtype, bias, act, kEpiStore, 0,
                  static_cast<cudaStream_t>(stream));
}

int sfb200_sparse_gemm_swiglu(const void* x, int ldx, const void* values_gu, const void* meta_gu,
                              void* h, int ldh, int M, int I, int K, int dtype, void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  Range r("sfb200.gate_up_gemm");
  return run_gemm(s, x, ldx, values_gu, meta_gu, h, ldh, M, 2 * I, K, dtype, nullptr, kActNone,
                  kEpiSwiGLU, 0, static_cast<cudaStream_t>(stream));
}

int sfb200_silu_mul(const void* gate, int ld_gate, const void* up, int ld_up, void* out, int ld_out,
                    int rows, int cols, int dtype, void* stream) {
  int err = kOk;
  if (!device_state(&err)) return err;
  return launch_silu_mul(gate, up, out, rows, cols, ld_gate, ld_up, ld_out, dtype,
                         static_cast<cudaStream_t>(stream));
}

int sfb200_ffn_forward(const sfb200_ffn_weights* w, const void* x, int ldx, void* hidden, void* out,
                       int ldo, int M, void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  if (!w || !hidden) return kErrInvalid;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc;
  {
    Range r("sfb200.gate_up_gemm");
    rc = run_gemm(s, x, ldx, w->gu_values, w->gu_meta, hidden, w->I, M, 2 * w->I, w->H, w->dtype,
                  nullptr, kActNone, kEpiSwiGLU, 0, st);
  }
  if (rc != kOk) return rc;
  Range r("sfb200.down_gemm");
  return run_gemm(s, hidden, w->I, w->down_values, w->down_meta, out, ldo, M, w->H, w->I, w->dtype,
                  w->down_bias, kActNone, kEpiStore, 0, st);
}

int sfb200_ffn_forward_host(const sfb200_ffn_weights* w, const void* x_host, void* out_host, int M,
                            void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  if (!w || !x_host || !out_host || M <= 0) return kErrInvalid;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t xb = static_cast<size_t>(M) * w->H * 2, hb = static_cast<size_t>(M) * w->I * 2;
  {
    std::lock_guard<std::mutex> lk(g_state_mu);
    if (s->stage_x_bytes < xb) {
      if (s->stage_x) cudaFree(s->stage_x);
      if (s->stage_o) cudaFree(s->stage_o);
      s->stage_x = s->stage_o = nullptr;
      s->stage_x_bytes = 0;
      if (cudaMalloc(&s->stage_x, xb) != cudaSuccess || cudaMalloc(&s->stage_o, xb) != cudaSuccess) {
        cudaGetLastError();
        return kErrOutOfMemory;
      }
      s->stage_x_bytes = xb;
    }
    if (s->stage_h_bytes < hb) {
      if (s->stage_h) cudaFree(s->stage_h);
      s->stage_h = nullptr;
      s->stage_h_bytes = 0;
      if (cudaMalloc(&s->stage_h, hb) != cudaSuccess) {
        cudaGetLastError();
        return kErrOutOfMemory;
      }
      s->stage_h_bytes = hb;
    }
  }
  // Pipeline over token chunks: host->device copy of chunk i+1, FFN of chunk i and device->host
  // copy of chunk i-1 run concurrently (copy-in stream, the caller's stream, copy-out stream).
  {
    std::lock_guard<std::mutex> lk(g_state_mu);
    if (!s->pipe_ready) {
      bool ok = cudaStreamCreateWithFlags(&s->s_in, cudaStreamNonBlocking) == cudaSuccess &&
                cudaStreamCreateWithFlags(&s->s_out, cudaStreamNonBlocking) == cudaSuccess &&
                cudaEventCreateWithFlags(&s->ev_start, cudaEventDisableTiming) == cudaSuccess &&
                cudaEventCreateWithFlags(&s->ev_done, cudaEventDisableTiming) == cudaSuccess;
      for (int i = 0; ok && i < DeviceState::kMaxChunks; ++i)
        ok = cudaEventCreateWithFlags(&s->ev_in[i], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&s->ev_cmp[i], cudaEventDisableTiming) == cudaSuccess;
      if (!ok) {
        cudaGetLastError();
        return kErrCuda;
      }
      s->pipe_ready = true;
    }
  }
  // Chunk plan: `main` rows per chunk while more than that remains, then the remainder is halved
  // down to `tail` rows.  The copy-in stream is the bottleneck (PCIe); what follows the last
  // copy-in -- FFN and copy-out of the LAST chunk -- is pure latency, but small chunks also run
  // the GEMMs less efficiently, so the default keeps the tail at the main size.
  int plan[DeviceState::kMaxChunks];
  const int n_chunks = plan_host_chunks(M, s->host_main_rows, s->host_tail_rows, plan);
  const size_t row_x = static_cast<size_t>(w->H) * 2, row_h = static_cast<size_t>(w->I) * 2;
  if (cudaEventRecord(s->ev_start, st) != cudaSuccess) return kErrCuda;
  if (cudaStreamWaitEvent(s->s_in, s->ev_start, 0) != cudaSuccess) return kErrCuda;
  if (cudaStreamWaitEvent(s->s_out, s->ev_start, 0) != cudaSuccess) return kErrCuda;
  int r0 = 0;
  for (int c = 0; c < n_chunks; r0 += plan[c], ++c) {
    const int rows = plan[c];
    uint8_t* xd = static_cast<uint8_t*>(s->stage_x) + r0 * row_x;
    uint8_t* od = static_cast<uint8_t*>(s->stage_o) + r0 * row_x;
    uint8_t* hd = static_cast<uint8_t*>(s->stage_h) + r0 * row_h;
    if (cudaMemcpyAsync(xd, static_cast<const uint8_t*>(x_host) + r0 * row_x, rows * row_x,
                        cudaMemcpyHostToDevice, s->s_in) != cudaSuccess)
      return kErrCuda;
    cudaEventRecord(s->ev_in[c], s->s_in);
    cudaStreamWaitEvent(st, s->ev_in[c], 0);
    const int rc = sfb200_ffn_forward(w, xd, w->H, hd, od, w->H, rows, stream);
    if (rc != kOk) return rc;
    cudaEventRecord(s->ev_cmp[c], st);
    cudaStreamWaitEvent(s->s_out, s->ev_cmp[c], 0);
    if (cudaMemcpyAsync(static_cast<uint8_t*>(out_host) + r0 * row_x, od, rows * row_x, cudaMemcpyDeviceToHost,
                        s->s_out) != cudaSuccess)
      return kErrCuda;
  }
  cudaEventRecord(s->ev_done, s->s_out);
  cudaStreamWaitEvent(st, s->ev_done, 0);
  if (cudaStreamSynchronize(st) != cudaSuccess) return kErrCuda;
  return kOk;
}

int sfb200_sparse_gemm_scatter(const void* x, int ldx, const void* values, const void* meta,
                               void* const* peer_slots, int tp, int rank, int tok_per_owner, int slots_f32, int M, int N, int K,
                               int dtype, void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  if (!x || !values || !meta || !peer_slots) return kErrInvalid;
  if (dtype != kF16 && dtype != kBF16) return kErrInvalid;
  Range r("sfb200.down_gemm_scatter");
  SparseGemmArgs a{};
  a.x = x;
  a.values = values;
  a.meta = meta;
  a.y = peer_slots[0];      // unused by the kernel when peer_y is set; kept non-null for the launch checks
  a.status = s->status;
  a.m_tok = M;
  a.n_out = N;
  a.K = K;
  a.ldx = ldx;
  a.ldy = N;
  a.fmt = dtype;
  a.epi = kEpiStore;
  a.act = kActNone;
  a.num_sms = s->num_sms;
  a.force_bn = s->force_bn;
  if (slots_f32 < 0 || slots_f32 > 2 || rank < 0 || rank >= tp) return kErrInvalid;
  a.out_f32 = slots_f32;
  a.peer_y = peer_slots;
  a.tp = tp;
  a.rank = rank;
  a.tok_per_owner = tok_per_owner;
  // a forced variant of another kernel family means nothing here: let the pair launcher choose (it keeps to the tiles
  // with two accumulator sets, whose drain -- here stores over NVLink -- hides behind the next tile's K loop)
  if (a.force_bn < 1000 || (a.force_bn >= 3000 && a.force_bn < 5000)) a.force_bn = 0;
  return launch_sparse_gemm_pair(a, static_cast<cudaStream_t>(stream));
}

int sfb200_sparse_gemm_f32out(const void* x, int ldx, const void* values, const void* meta, float* y, int ldy, int M,
                              int N, int K, int dtype, const void* bias, int act, void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  if (!x || !values || !meta || !y) return kErrInvalid;
  if (dtype != kF16 && dtype != kBF16) return kErrInvalid;
  Range r("sfb200.sparse_gemm_f32out");
  SparseGemmArgs a{};
  a.x = x;
  a.values = values;
  a.meta = meta;
  a.y = y;
  a.bias = bias;
  a.status = s->status;
  a.m_tok = M;
  a.n_out = N;
  a.K = K;
  a.ldx = ldx;
  a.ldy = ldy;
  a.fmt = dtype;
  a.epi = kEpiStore;
  a.act = act;
  a.num_sms = s->num_sms;
  a.force_bn = s->force_bn;
  a.out_f32 = 1;
  return launch_sparse_gemm(a, static_cast<cudaStream_t>(stream));
}

int sfb200_tp_push_reduce(const void* partial_chunk, int block_rows, const int* valid_rows, void* const* peer_slots,
                          const void* slots, int slot_rows, int slots_f32, void* const* peer_out_blocks, int rows, int cols,
                          int dtype, const void* bias, void* const* peer_flags, int tp, int rank, unsigned epoch, int light,
                          void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  if (!partial_chunk || !valid_rows || !peer_slots || tp < 2 || tp > 8) return kErrInvalid;
  Range r("sfb200.tp_push_reduce");
  ExchangePush push = {};
  push.src = partial_chunk;
  push.peer_slots = peer_slots;
  push.block_rows = block_rows;
  for (int o = 0; o < tp; ++o) push.valid_rows[o] = valid_rows[o];
  push.light = light;
  return launch_exchange(3, slots, nullptr, peer_out_blocks, rows, cols, slot_rows, slots_f32, dtype, bias, peer_flags, tp,
                         rank, epoch, s->status, static_cast<cudaStream_t>(stream), &push);
}

int sfb200_tp_allreduce_switch(const void* mc_partial_block, void* mc_out_block, int rows, int cols, int dtype,
                               int partial_f32, const void* bias, void* const* peer_flags, int tp, int rank,
                               unsigned epoch, void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  Range r("sfb200.tp_allreduce_switch");
  return launch_exchange(partial_f32 ? 2 : 1, mc_partial_block, mc_out_block, nullptr, rows, cols, rows, partial_f32, dtype,
                         bias, peer_flags, tp, rank, epoch, s->status, static_cast<cudaStream_t>(stream));
}

int sfb200_tp_allgather(const void* local_block, void* mc_dst_block, void* const* peer_dst_blocks, int rows, int cols,
                        void* const* peer_flags, int tp, int rank, unsigned epoch, void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  Range r("sfb200.tp_allgather");
  return launch_exchange(0, local_block, mc_dst_block, peer_dst_blocks, rows, cols, rows, 0, kBF16, nullptr, peer_flags, tp,
                         rank, epoch, s->status, static_cast<cudaStream_t>(stream));
}

int sfb200_tp_reduce_slots(const void* slots, int slot_rows, int slots_f32, void* mc_out_block, void* const* peer_out_blocks,
                           int rows, int cols, int dtype, const void* bias, void* const* peer_flags, int tp, int rank,
                           unsigned epoch, void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  Range r("sfb200.tp_reduce_slots");
  return launch_exchange(3, slots, mc_out_block, peer_out_blocks, rows, cols, slot_rows, slots_f32, dtype, bias, peer_flags,
                         tp, rank, epoch, s->status, static_cast<cudaStream_t>(stream));
}

int sfb200_tp_flag_words(void) { return kSwitchFlagWords; }

/* Test / tuning hook: force the token tile of the tcgen05 kernel (0 = automatic). */
SFB200_API int sfb200_debug_force_token_tile(int bn) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  s->force_bn = bn;
  return kOk;
}

SFB200_API int sfb200_debug_pair_tuning(int l2_band_mb, int force_order) {
  if (force_order < -1 || force_order > 1) return kErrInvalid;
  set_pair_tuning(l2_band_mb, force_order);
  return kOk;
}

/* Which kernel variant sfb200_sparse_gemm (swiglu = 0) or sfb200_sparse_gemm_swiglu (swiglu = 1, N = 2 * I
 * rows) runs for a shape on a GPU with num_sms SMs, in the numbering of sfb200_debug_force_token_tile.  Host-only. */
SFB200_API int sfb200_debug_plan_gemm(int M, int N, int K, int swiglu, int num_sms) {
  if (M <= 0 || N <= 0 || K <= 0 || num_sms <= 0) return 0;
  return plan_sparse_gemm(M, N, K, swiglu ? kEpiSwiGLU : kEpiStore, num_sms);
}

/* The chunk plan sfb200_ffn_forward_host would use for M tokens (host-only; out8 holds 8 ints). */
SFB200_API int sfb200_debug_host_chunk_plan(int M, int main_rows, int tail_rows, int* out8) {
  if (M <= 0 || !out8) return 0;
  return plan_host_chunks(M, main_rows, tail_rows, out8);
}

/* Tuning hook: rows per main chunk / smallest tail chunk of sfb200_ffn_forward_host (0 = default). */
SFB200_API int sfb200_debug_host_pipeline(int main_rows, int tail_rows) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  s->host_main_rows = main_rows;
  s->host_tail_rows = tail_rows;
  return kOk;
}

}  // extern "C"
