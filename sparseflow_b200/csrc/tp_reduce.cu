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

// ---------------------------------------------------------------- exchange through NVSwitch, one kernel
//
// The whole exchange step of the row-parallel GEMM in ONE launch per rank: every rank has written its
// partial output [M, cols] into its own copy of a symmetric buffer; this kernel waits until all ranks
// have done so, sums its own token block ACROSS ranks inside the switch (multimem.ld_reduce, fp32
// accumulation of the 16-bit partials), adds the bias, rounds once and writes the finished block
// into every rank's output with multimem.st, then waits until every rank has finished.  Compared
// with "scatter in the GEMM epilogue + barrier + reduce kernel + barrier" it moves the same bytes
// out of each GPU but needs one launch instead of four and reads 1/tp of the partials instead of
// all of them through this GPU's memory.
//
// Cross-GPU ordering uses flag words in symmetric memory, one set per CTA: CTA b of rank r stores
// the launch's epoch into slot [b][r] of every rank (st.release.sys) and polls its own slots
// [b][0..tp) (ld.acquire.sys) -- CTA b talks only to CTA b of the other ranks, so every rank must
// launch the same grid.  Epochs increase by one per launch and are never reset.  Every poll loop is
// bounded: after kPeerWaitLimitNs it records (2 << 8) | phase in the status word, the CTA skips its
// remaining work and waits, and the kernel returns.
// No load of any kind names a peer's memory directly; the multicast address is the only remote path.
constexpr unsigned long long kPeerWaitLimitNs = 2000000000ull;
constexpr int kExchangeCtas = 148;
constexpr int kExchangeThreads = 512;
constexpr int kStatusPeerTimeout = 2;

struct FlagPeers {
  uint32_t* p[8];   // each rank's flag array (peer-mapped); [0, ctas*8) entry flags, [ctas*8, 2*ctas*8) exit flags
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Threads 0..tp-1 of the CTA: announce `epoch` in slot [cta][rank] of every rank, then wait until all
// of this rank's slots [cta][0..tp) have reached it.  Returns false (warp-uniform per thread) on timeout.
__device__ __forceinline__ bool cta_rank_barrier(const FlagPeers& peers, uint32_t* local, int region_off, int tp,
                                                 int rank, uint32_t epoch, int* status, int phase,
                                                 unsigned long long limit_ns) {
  const int t = threadIdx.x;
  bool ok = true;
  if (t < tp) {
    const int slot = region_off + blockIdx.x * 8;
    st_release_sys(peers.p[t] + slot + rank, epoch);
    const uint32_t* mine = local + slot + t;
    const unsigned long long t0 = timer_ns();
    // signed distance: epochs only grow, a peer may already be one launch ahead
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (timer_ns() - t0 > limit_ns) {
        atomicCAS(status, 0, (kStatusPeerTimeout << 8) | phase);
        ok = false;
        break;
      }
    }
  }
  return ok;
}

template <bool BF16, bool REDUCE>
__global__ void __launch_bounds__(kExchangeThreads, 1)
switch_exchange_kernel(const uint4* src, uint4* mc_dst, size_t vec, int vec_per_row, const uint16_t* bias, FlagPeers peers,
                       uint32_t* local_flags, int tp, int rank, uint32_t epoch, int* status, unsigned long long limit_ns) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  // ---- every rank's source data is complete (its producer kernel precedes this one on its stream)
  if (!cta_rank_barrier(peers, local_flags, 0, tp, rank, epoch, status, 1, limit_ns)) failed = 1;
  __syncthreads();
  if (!failed) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i0 < vec; i0 += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t i = i0 + u * stride;
        if (i < vec) {
          if (REDUCE) {
            if (BF16)
              asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                           : "l"(src + i)
                           : "memory");
            else
              asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                           : "l"(src + i)
                           : "memory");
          } else {
            v[u] = __ldg(src + i);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t i = i0 + u * stride;
        if (i < vec) {
          uint4 o = v[u];
          if (REDUCE && bias) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            add8<BF16>(acc, o);
            const int c0 = static_cast<int>(i % vec_per_row) * 8;
            uint32_t* ow = &o.x;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float a = acc[2 * j], b = acc[2 * j + 1];
              if (BF16) {
                a += __uint_as_float(static_cast<uint32_t>(bias[c0 + 2 * j]) << 16);
                b += __uint_as_float(static_cast<uint32_t>(bias[c0 + 2 * j + 1]) << 16);
                const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                ow[j] = *reinterpret_cast<const uint32_t*>(&h);
              } else {
                a += __half2float(__ushort_as_half(bias[c0 + 2 * j]));
                b += __half2float(__ushort_as_half(bias[c0 + 2 * j + 1]));
                const __half2 h = __floats2half2_rn(a, b);
                ow[j] = *reinterpret_cast<const uint32_t*>(&h);
              }
            }
          }
          store_all_ranks(mc_dst + i, o);
        }
      }
    }
  }
  // ---- this CTA's stores are ordered before its exit flag; then every rank has finished
  __threadfence_system();
  __syncthreads();
  if (!failed) cta_rank_barrier(peers, local_flags, kExchangeCtas * 8, tp, rank, epoch, status, 2, limit_ns);
}

}  // namespace

int launch_switch_exchange(bool reduce, const void* src, void* mc_dst, int rows, int cols, int fmt, const void* bias,
                           void* const* peer_flags, int tp, int rank, unsigned epoch, int* status, cudaStream_t stream) {
  // rows == 0: this rank contributes no block but still takes part in the two barriers
  if (!src || !mc_dst || !peer_flags || !status || rows < 0 || cols <= 0 || cols % 8 != 0) return kErrInvalid;
  if (tp < 2 || tp > 8 || rank < 0 || rank >= tp || epoch == 0) return kErrInvalid;
  if (fmt != kF16 && fmt != kBF16) return kErrInvalid;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(mc_dst)) & 15) return kErrInvalid;
  if (!reduce && bias) return kErrInvalid;
  FlagPeers peers = {};
  for (int d = 0; d < 8; ++d) {
    void* q = peer_flags[d < tp ? d : 0];
    if (!q || (reinterpret_cast<uintptr_t>(q) & 3)) return kErrInvalid;
    peers.p[d] = static_cast<uint32_t*>(q);
  }
  uint32_t* local = peers.p[rank];
  const size_t vec = static_cast<size_t>(rows) * cols / 8;
  const uint4* s4 = static_cast<const uint4*>(src);
  uint4* d4 = static_cast<uint4*>(mc_dst);
  const uint16_t* b16 = static_cast<const uint16_t*>(bias);
  if (reduce) {
    if (fmt == kBF16)
      switch_exchange_kernel<true, true><<<kExchangeCtas, kExchangeThreads, 0, stream>>>(
          s4, d4, vec, cols / 8, b16, peers, local, tp, rank, epoch, status, kPeerWaitLimitNs);
    else
      switch_exchange_kernel<false, true><<<kExchangeCtas, kExchangeThreads, 0, stream>>>(
          s4, d4, vec, cols / 8, b16, peers, local, tp, rank, epoch, status, kPeerWaitLimitNs);
  } else {
    switch_exchange_kernel<true, false><<<kExchangeCtas, kExchangeThreads, 0, stream>>>(
        s4, d4, vec, cols / 8, nullptr, peers, local, tp, rank, epoch, status, kPeerWaitLimitNs);
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

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
