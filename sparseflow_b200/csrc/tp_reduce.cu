// Second half of the fused tensor-parallel down projection.  After every rank's GEMM epilogue has
// stored its partial sums of token block r into rank r's receive slots (one slot per source rank),
// rank r adds the slots in fp32 and writes the finished block into the output tensor of EVERY rank
// : the all-gather is fused into the reduction, so the partial sums cross NVLink once and the
// finished block once.  The finished block is written either with plain 16-byte stores to each rank's
// peer-mapped memory (tp - 1 copies leave this GPU) or, when the output tensor has a switch-replicated
// mapping, with multimem.st (one copy leaves this GPU and NVSwitch fans it out).
// HBM / NVLink bound: reads tp * rows * cols * 2 B locally, writes rows * cols * 2 B to each rank.
// No kernel here waits on another GPU: ordering is by stream-ordered barriers between launches.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace sfb200 {
namespace {

struct PeerOut {
  uint4* p[8];
};

template <bool BF16>
__device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (BF16) {
      acc[2 * i] += __uint_as_float(w[i] << 16);
      acc[2 * i + 1] += __uint_as_float(w[i] & 0xFFFF0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      const float2 f = __half22float2(h);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
}

// One 16-byte store that NVSwitch replicates into the same offset of every rank's buffer (`mc` is an
// address inside the switch-replicated mapping of the symmetric output tensor).
__device__ __forceinline__ void store_all_ranks(uint4* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

template <bool BF16>
__global__ void __launch_bounds__(256) reduce_allgather_kernel(const uint4* slots, int tp, size_t vec_per_slot,
                                                               int vec_per_row, PeerOut out, uint4* mc_out,
                                                               const uint16_t* bias) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < vec_per_slot;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < tp; ++s) add8<BF16>(acc, __ldg(slots + s * vec_per_slot + i));
    if (bias) {
      const int c0 = static_cast<int>(i % vec_per_row) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        acc[j] += BF16 ? __uint_as_float(static_cast<uint32_t>(bias[c0 + j]) << 16)
                       : __half2float(__ushort_as_half(bias[c0 + j]));
    }
    uint4 o;
    uint32_t* ow = &o.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        ow[j] = *reinterpret_cast<const uint32_t*>(&v);
      } else {
        const __half2 v = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
        ow[j] = *reinterpret_cast<const uint32_t*>(&v);
      }
    }
    if (mc_out != nullptr) store_all_ranks(mc_out + i, o);     // the block leaves this GPU once
    else
      for (int d = 0; d < tp; ++d) out.p[d][i] = o;
  }
}

}  // namespace

int launch_reduce_allgather(const void* slots, int tp, int rows, int cols, void* const* peer_out_blocks,
                            void* switch_out_block, int fmt, const void* bias, cudaStream_t stream) {
  if (!slots || tp < 1 || tp > 8 || rows <= 0 || cols <= 0 || cols % 8 != 0) return kErrInvalid;
  if (fmt != kF16 && fmt != kBF16) return kErrInvalid;
  if (!peer_out_blocks && !switch_out_block) return kErrInvalid;
  if (reinterpret_cast<uintptr_t>(switch_out_block) & 15) return kErrInvalid;
  PeerOut out = {};
  for (int d = 0; d < 8 && switch_out_block == nullptr; ++d) {
    void* q = peer_out_blocks[d < tp ? d : 0];
    if (!q || (reinterpret_cast<uintptr_t>(q) & 15)) return kErrInvalid;
    out.p[d] = static_cast<uint4*>(q);
  }
  const size_t vec = static_cast<size_t>(rows) * cols / 8;
  size_t blocks = (vec + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (fmt == kBF16)
    reduce_allgather_kernel<true><<<static_cast<int>(blocks), 256, 0, stream>>>(
        static_cast<const uint4*>(slots), tp, vec, cols / 8, out, static_cast<uint4*>(switch_out_block),
        static_cast<const uint16_t*>(bias));
  else
    reduce_allgather_kernel<false><<<static_cast<int>(blocks), 256, 0, stream>>>(
        static_cast<const uint4*>(slots), tp, vec, cols / 8, out, static_cast<uint4*>(switch_out_block),
        static_cast<const uint16_t*>(bias));
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

}  // namespace sfb200
