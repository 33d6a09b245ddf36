// Exchange kernels of the tensor-parallel FFN: the reduction of the row-parallel GEMM's partial sums across ranks
// and the replication of the finished token blocks, one launch per rank, over NVLink peer stores or through
// NVSwitch (multimem).  HBM / NVLink bound.
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

// ---------------------------------------------------------------- exchange step, one kernel per rank
//
// The reduction + all-gather of the row-parallel GEMM in ONE launch per rank, with the cross-GPU ordering inside the
// kernel.  Four forms (MODE):
//   3  "push": every rank's GEMM epilogue has already stored its partial sums of token block r into rank r's receive
//      slots (one slot per source rank, local memory here).  This kernel waits until all ranks' GEMMs are done, adds
//      the tp slots in fp32 (slots are FLOAT or 16-bit), adds the bias, rounds ONCE and stores the finished block
//      into every rank's output with plain 16-byte peer stores (or one multimem.st when a switch-replicated mapping
//      of the output is given).  Needs no multicast support.
//   1/2 "pull through the switch": every rank wrote its partial output into its own copy of a symmetric buffer; this
//      rank's block is summed across ranks inside NVSwitch (multimem.ld_reduce; 16-bit partials with fp32
//      accumulation, or FLOAT partials) and written to every rank with multimem.st.
//   0  all-gather of one local 16-bit block per rank (e.g. the activations each rank uploaded).
// Every form returns only when every rank has finished, so the caller's next kernel may overwrite the buffers.
//
// Cross-GPU ordering uses flag words in symmetric memory, one set per CTA: CTA b of rank r stores the launch's epoch
// into slot [b][r] of every rank (st.release.sys) and polls its own slots [b][0..tp) (ld.acquire.sys) -- CTA b
// talks only to CTA b of the other ranks, so every rank launches the same grid.  Epochs increase by one per launch
// and are never reset.  Every poll loop is bounded: after kPeerWaitLimitNs it records (2 << 8) | phase in the
// status word, the CTA skips its remaining work and waits, and the kernel returns.
// No load of any kind names a peer's memory directly: remote data arrives by peers' stores or through multimem.
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
// of this rank's slots [cta][0..tp) have reached it.  Returns false on timeout.
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

template <bool BF16>
__device__ __forceinline__ uint4 round8(const float (&acc)[8]) {
  uint4 o;
  uint32_t* ow = &o.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (BF16) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      ow[j] = *reinterpret_cast<const uint32_t*>(&h);
    } else {
      const __half2 h = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
      ow[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  return o;
}

struct ExchangeArgs {
  const void* src;        // MODE 0: local block; 1/2: multicast address of the block; 3: local slots [tp][slot_units]
  uint4* mc_dst;          // multicast address of the destination block, or null (MODE 0 / 3: peer stores instead)
  PeerOut out;            // destination block in every rank's buffer (used when mc_dst is null)
  size_t vec;             // 16-byte units of OUTPUT (8 values each) in the block
  size_t slot_units;      // MODE 3: distance between two source ranks' slots, in output units
  int vec_per_row;
  int slots_f32;          // MODE 3: slots hold floats
  int slots_half;         // MODE 3: slots hold fp16 whatever the output type
  const uint16_t* bias;
  FlagPeers peers;
  uint32_t* local_flags;
  int tp, rank;
  uint32_t epoch;
  int* status;
  unsigned long long limit_ns;
  // MODE 3, optional push phase before the entry barrier (the reduce-scatter as a copy, for GEMMs that wrote their
  // partial sums locally): owner block o of push_src ([tp][push_block_units] units apart, push_valid_units[o] of them
  // live) is copied to push_dst.p[o], the slot that rank o keeps for this rank
  const void* push_src;
  PeerOut push_dst;
  size_t push_block_units;
  unsigned push_valid_units[8];
};

// LIGHT = 128 threads and at most 85 registers: fits on an SM BESIDE a GEMM CTA (320 threads, 54 K registers), so the
// exchange of one token chunk can run while the GEMMs of the next chunk do.
template <bool BF16, int MODE, bool LIGHT>
__global__ void __launch_bounds__(LIGHT ? 128 : kExchangeThreads, LIGHT ? 6 : 1) exchange_kernel(const ExchangeArgs a) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (MODE == 3 && a.push_src != nullptr) {
    // same element <-> (CTA, thread) mapping as the reduction below: what CTA b of rank o reduces was pushed by
    // CTA b of every rank, so the per-CTA barrier that follows is all the ordering the data needs
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const int per_unit = a.slots_f32 ? 2 : 1;     // 16-byte pieces per output unit
    for (int o = 0; o < a.tp; ++o) {
      const uint4* src = static_cast<const uint4*>(a.push_src) + static_cast<size_t>(o) * a.push_block_units * per_unit;
      uint4* dst = a.push_dst.p[o];
      const size_t n = a.push_valid_units[o];
      for (size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i0 < n; i0 += 4 * stride) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const size_t i = i0 + u * stride;
          if (i < n) {
            v[2 * u] = __ldcs(src + per_unit * i);
            if (per_unit == 2) v[2 * u + 1] = __ldcs(src + 2 * i + 1);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const size_t i = i0 + u * stride;
          if (i < n) {
            dst[per_unit * i] = v[2 * u];
            if (per_unit == 2) dst[2 * i + 1] = v[2 * u + 1];
          }
        }
      }
    }
    __threadfence_system();
    __syncthreads();
  }
  // ---- every rank's source data is complete (its producer kernel precedes this one on its stream)
  if (!cta_rank_barrier(a.peers, a.local_flags, 0, a.tp, a.rank, a.epoch, a.status, 1, a.limit_ns)) failed = 1;
  __syncthreads();
  if (!failed) {
    constexpr int U = (MODE == 3) ? 1 : 4;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i0 < a.vec; i0 += U * stride) {
      uint4 v[U], w[U];
      float acc3[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t i = i0 + u * stride;
        if (i >= a.vec) continue;
        if (MODE == 3) {
          // four slots' loads are issued before their adds (local HBM / L2 reads), twice
          if (a.slots_f32) {
            const uint4* s = static_cast<const uint4*>(a.src) + 2 * i;
#pragma unroll
            for (int r0 = 0; r0 < 8; r0 += 4) {
              uint4 x0[4], x1[4];
#pragma unroll
              for (int r = 0; r < 4; ++r)
                if (r0 + r < a.tp) {
                  x0[r] = __ldcs(s + 2 * (r0 + r) * a.slot_units);
                  x1[r] = __ldcs(s + 2 * (r0 + r) * a.slot_units + 1);
                }
#pragma unroll
              for (int r = 0; r < 4; ++r)
                if (r0 + r < a.tp) {
                  acc3[0] += __uint_as_float(x0[r].x); acc3[1] += __uint_as_float(x0[r].y);
                  acc3[2] += __uint_as_float(x0[r].z); acc3[3] += __uint_as_float(x0[r].w);
                  acc3[4] += __uint_as_float(x1[r].x); acc3[5] += __uint_as_float(x1[r].y);
                  acc3[6] += __uint_as_float(x1[r].z); acc3[7] += __uint_as_float(x1[r].w);
                }
            }
          } else {
            const uint4* s = static_cast<const uint4*>(a.src) + i;
            uint4 x0[8];
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (r < a.tp) x0[r] = __ldcs(s + r * a.slot_units);
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (r < a.tp) {
                if (a.slots_half) add8<false>(acc3, x0[r]);
                else add8<BF16>(acc3, x0[r]);
              }
          }
        } else if (MODE == 2) {
          const uint4* s = static_cast<const uint4*>(a.src) + 2 * i;
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                       : "l"(s)
                       : "memory");
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(w[u].x), "=r"(w[u].y), "=r"(w[u].z), "=r"(w[u].w)
                       : "l"(s + 1)
                       : "memory");
        } else if (MODE == 1) {
          const uint4* s = static_cast<const uint4*>(a.src) + i;
          if (BF16)
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                         : "l"(s)
                         : "memory");
          else
            asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                         : "l"(s)
                         : "memory");
        } else {
          v[u] = __ldg(static_cast<const uint4*>(a.src) + i);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t i = i0 + u * stride;
        if (i >= a.vec) continue;
        uint4 o = v[u];
        if (MODE >= 2 || (MODE == 1 && a.bias)) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (MODE == 3) {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = acc3[j];
          } else if (MODE == 2) {
            const uint32_t f[8] = {v[u].x, v[u].y, v[u].z, v[u].w, w[u].x, w[u].y, w[u].z, w[u].w};
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = __uint_as_float(f[j]);
          } else {
            add8<BF16>(acc, o);
          }
          if (a.bias) {
            const int c0 = static_cast<int>(i % a.vec_per_row) * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              acc[j] += BF16 ? __uint_as_float(static_cast<uint32_t>(a.bias[c0 + j]) << 16)
                             : __half2float(__ushort_as_half(a.bias[c0 + j]));
          }
          o = round8<BF16>(acc);
        }
        if (a.mc_dst != nullptr) store_all_ranks(a.mc_dst + i, o);
        else {
#pragma unroll
          for (int d = 0; d < 8; ++d)
            if (d < a.tp) a.out.p[d][i] = o;
        }
      }
    }
  }
  // ---- this CTA's stores are ordered before its exit flag; then every rank has finished
  __threadfence_system();
  __syncthreads();
  if (!failed) cta_rank_barrier(a.peers, a.local_flags, kExchangeCtas * 8, a.tp, a.rank, a.epoch, a.status, 2, a.limit_ns);
}

}  // namespace

int launch_exchange(int mode, const void* src, void* mc_dst, void* const* peer_dst, int rows, int cols, int slot_rows,
                    int slots_f32, int fmt, const void* bias, void* const* peer_flags, int tp, int rank, unsigned epoch,
                    int* status, cudaStream_t stream, const ExchangePush* push) {
  // rows == 0: this rank contributes no block but still takes part in the two barriers
  if (!src || !peer_flags || !status || rows < 0 || cols <= 0 || cols % 8 != 0) return kErrInvalid;
  if (!mc_dst && !peer_dst) return kErrInvalid;
  if (tp < 2 || tp > 8 || rank < 0 || rank >= tp || epoch == 0 || mode < 0 || mode > 3) return kErrInvalid;
  if (fmt != kF16 && fmt != kBF16) return kErrInvalid;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(mc_dst)) & 15) return kErrInvalid;
  if (mode == 0 && bias) return kErrInvalid;
  if ((mode == 1 || mode == 2) && !mc_dst) return kErrInvalid;
  if (mode == 3 && slot_rows < rows) return kErrInvalid;
  if (push && mode != 3) return kErrInvalid;
  ExchangeArgs a = {};
  for (int d = 0; d < 8; ++d) {
    void* q = peer_flags[d < tp ? d : 0];
    if (!q || (reinterpret_cast<uintptr_t>(q) & 3)) return kErrInvalid;
    a.peers.p[d] = static_cast<uint32_t*>(q);
    if (!mc_dst) {
      void* o = peer_dst[d < tp ? d : 0];
      if (!o || (reinterpret_cast<uintptr_t>(o) & 15)) return kErrInvalid;
      a.out.p[d] = static_cast<uint4*>(o);
    }
  }
  a.src = src;
  a.mc_dst = static_cast<uint4*>(mc_dst);
  a.vec = static_cast<size_t>(rows) * cols / 8;
  a.slot_units = static_cast<size_t>(slot_rows) * cols / 8;
  a.vec_per_row = cols / 8;
  if (slots_f32 < 0 || slots_f32 > 2 || (slots_f32 == 2 && mode != 3)) return kErrInvalid;
  a.slots_f32 = slots_f32 == 1;
  a.slots_half = slots_f32 == 2;
  a.bias = static_cast<const uint16_t*>(bias);
  a.local_flags = a.peers.p[rank];
  a.tp = tp;
  a.rank = rank;
  a.epoch = epoch;
  a.status = status;
  a.limit_ns = kPeerWaitLimitNs;
  bool light = false;
  if (push) {
    if (!push->src || push->block_rows <= 0 || (reinterpret_cast<uintptr_t>(push->src) & 15)) return kErrInvalid;
    a.push_src = push->src;
    a.push_block_units = static_cast<size_t>(push->block_rows) * cols / 8;
    for (int o = 0; o < 8; ++o) {
      void* q = push->peer_slots[o < tp ? o : 0];
      if (!q || (reinterpret_cast<uintptr_t>(q) & 15)) return kErrInvalid;
      a.push_dst.p[o] = static_cast<uint4*>(q);
      const int valid = o < tp ? push->valid_rows[o] : 0;
      if (valid < 0 || valid > push->block_rows) return kErrInvalid;
      a.push_valid_units[o] = static_cast<unsigned>(static_cast<size_t>(valid) * cols / 8);
    }
    light = push->light != 0;
  }
  const bool bf = fmt == kBF16;
#define SFB_LAUNCH_EXCHANGE(BF, MODE) exchange_kernel<BF, MODE, false><<<kExchangeCtas, kExchangeThreads, 0, stream>>>(a)
  if (mode == 0) SFB_LAUNCH_EXCHANGE(true, 0);
  else if (mode == 1 && bf) SFB_LAUNCH_EXCHANGE(true, 1);
  else if (mode == 1) SFB_LAUNCH_EXCHANGE(false, 1);
  else if (mode == 2 && bf) SFB_LAUNCH_EXCHANGE(true, 2);
  else if (mode == 2) SFB_LAUNCH_EXCHANGE(false, 2);
  else if (light && bf) exchange_kernel<true, 3, true><<<kExchangeCtas, 128, 0, stream>>>(a);
  else if (light) exchange_kernel<false, 3, true><<<kExchangeCtas, 128, 0, stream>>>(a);
  else if (bf) SFB_LAUNCH_EXCHANGE(true, 3);
  else SFB_LAUNCH_EXCHANGE(false, 3);
#undef SFB_LAUNCH_EXCHANGE
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

}  // namespace sfb200
