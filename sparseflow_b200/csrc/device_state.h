// Per-device library state: status word, device facts, staging buffers of the host-buffer FFN call.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include <atomic>

namespace sfb200 {

constexpr int kMaxDevices = 16;

struct DeviceState {
  std::atomic<bool> ready{false};
  int cc = 0;
  int num_sms = 0;
  size_t total_mem = 0;
  int* status = nullptr;       // device status word (256-byte allocation, word 0 used)
  int force_bn = 0;            // tuning hook: token tile override
  void* stage_x = nullptr;     // host-buffer FFN: device copies of x / out, hidden scratch
  void* stage_o = nullptr;
  void* stage_h = nullptr;
  size_t stage_x_bytes = 0;
  size_t stage_h_bytes = 0;
  // host-buffer FFN pipeline: copy-in / copy-out streams and per-chunk events
  static constexpr int kMaxChunks = 8;
  int host_main_rows = 0, host_tail_rows = 0;  // chunk plan overrides of the host-buffer pipeline (0 = default)
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t ev_start = nullptr, ev_done = nullptr;
  cudaEvent_t ev_in[kMaxChunks] = {}, ev_cmp[kMaxChunks] = {};
  bool pipe_ready = false;
};

// State of the current device, created on first use.  Returns nullptr and sets *err when there is
// no usable sm_100 device.
DeviceState* device_state(int* err);

// Status word of sfb200_ffn_forward_noalloc on the current device (it lives in the library image, not in
// DeviceState): synchronises, reads and clears it; *word = 0 when that entry point never ran here.
int noalloc_take_status(int* word);
int* noalloc_status_word();   // its device address (sets the entry point up on the current device), or nullptr

}  // namespace sfb200
