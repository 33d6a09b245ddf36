// 2:4-sparse GEMM for sm_100a, CTA-pair variant for prefill-sized token counts.
//
// Same math and operand formats as sparse_gemm_sm100.cu, but two CTAs (a cluster of 2, on an SM
// pair) work on one 256-row x 256-token tile with tcgen05.mma.sp.cta_group::2:
//   * each CTA holds 128 weight rows (its own compressed values + metadata tile) and HALF of the
//     token tile, so per MMA an SM reads 4 KiB of A + 8 KiB of B from shared memory instead of
//     4 + 16: this is what lifts the single-CTA kernel's shared-memory and L2 bandwidth bound
//     (tile intensity 2RT/(R+2T) = 171 flop/B against 96-102 for 128x192/256);
//   * the even CTA of the pair issues every MMA; completion is signalled to both CTAs;
//   * the accumulator is 128 lanes x 256 fp32 columns per CTA and single-buffered (tensor memory
//     has 512 columns and the metadata needs some), so the epilogue drains it fast: 8 warps pull
//     their 128 columns into packed 16-bit registers, hand the accumulator back, and only then
//     write to global memory while the next tile's main loop is already running.
//
// 10 warps: warp 0 = TMA producer, warp 1 = MMA issuer / tensor-memory owner, warps 2..9 = epilogue.
// All loads are plain per-CTA TMA copies; nothing here reads another GPU's memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace sfb200 {

namespace {

// ---------------------------------------------------------------- cluster / pair PTX
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// Pair forms: the copy lands in this CTA's shared memory, the byte count is credited to the
// barrier of the even CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int x, int y,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_1d_pair(uint32_t dst, const CUtensorMap* m, int x,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.1d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2}], [%3];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// Arrive on the barrier at the same shared-memory offset in both CTAs of the pair once every
// tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}
__device__ __forceinline__ void tc_cp_128x128b_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_sp_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                   uint32_t e_tmem, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.sp.cta_group::2.kind::f16 [%0], %1, %2, [%3], %4, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct PairParams {
  const void* bias;
  void* y;
  int* status;
  int n_out, m_tok, K, ldy;
  int num_m_blks, num_n_blks;   // 256-row / BN-token tiles
  int k_tiles128;
  int fmt, act;
};

template <int BN_, int BK_, int STAGES_, int EPI_>
struct PairCfg {
  static constexpr int BN = BN_;         // tokens per tile (pair-wide)
  static constexpr int BK = BK_;
  static constexpr int STAGES = STAGES_;
  static constexpr int EPI = EPI_;
  static constexpr int HALF_N = BN / 2;  // tokens loaded by each CTA
  static constexpr int A_BYTES = 128 * (BK / 2) * 2;
  static constexpr int B_SUBS = BK / 64;
  static constexpr int B_SUB_BYTES = HALF_N * 128;
  static constexpr int B_BYTES = B_SUBS * B_SUB_BYTES;
  static constexpr int E_BYTES = 2048;
  static constexpr int MMAS_PER_STAGE = BK / 32;
  static constexpr int E_COL0 = BN;      // metadata columns start after the accumulator
  static constexpr int TMEM_USED = BN + 4 * STAGES;
  static constexpr int TMEM_COLS = TMEM_USED <= 128 ? 128 : TMEM_USED <= 256 ? 256 : 512;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_E = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_BAR = OFF_E + STAGES * E_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int EPI_WARPS = 8;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int COLS_PER_WARP = BN / 2;   // two warps share a lane quadrant
  static_assert(BN % 64 == 0 && BN <= 256, "BN");
  static_assert(TMEM_USED <= 512, "tmem");
  static_assert(SMEM_BYTES <= 232448, "smem");
};

__device__ __forceinline__ float act_fn(float v, int act) {
  switch (act) {
    case kActRelu: return fmaxf(v, 0.f);
    case kActSilu: return v * __fdividef(1.f, 1.f + __expf(-v));
    case kActGelu: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    default: return v;
  }
}
__device__ __forceinline__ uint32_t pack2(float a, float b, int fmt) {
  if (fmt == 1) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float bias_at(const void* bias, int o, int fmt) {
  const uint16_t b = static_cast<const uint16_t*>(bias)[o];
  if (fmt == 1) return __uint_as_float(static_cast<uint32_t>(b) << 16);
  return __half2float(__ushort_as_half(b));
}

template <class C>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(C::THREADS, 1)
sparse_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmE, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  const uint32_t bar_full = smem_u32(bars);                 // used in the even CTA only
  const uint32_t bar_empty = bar_full + 8 * C::STAGES;      // both CTAs
  const uint32_t bar_accf = bar_empty + 8 * C::STAGES;      // both CTAs
  const uint32_t bar_acce = bar_accf + 8;                   // even CTA only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + 8 * (2 * C::STAGES + 2));
  volatile int* err = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = p.num_m_blks * p.num_n_blks;
  const int k_iters = (p.K + C::BK - 1) / C::BK;

  if (threadIdx.x == 0) {
    *err = 0;
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_accf, 1);
    mbar_init(bar_acce, 2 * C::EPI_WARPS);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmE);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before anything remote touches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      const uint32_t leader_full0 = mapa_u32(bar_full, 0);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        const int m_blk = tile / p.num_n_blks;
        const int n_blk = tile % p.num_n_blks;
        const int row0 = m_blk * 256 + static_cast<int>(rank) * 128;
        const int tok0 = n_blk * C::BN + static_cast<int>(rank) * C::HALF_N;
        const int e_tile0 = (m_blk * 2 + static_cast<int>(rank)) * p.k_tiles128;
        for (int kt = 0; kt < k_iters; ++kt) {
          ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, err, p.status, 1);
          if (!ok) break;
          const bool load_e = (C::BK == 128) || ((kt & 1) == 0);
          const uint32_t full = leader_full0 + 8 * s;
          if (leader) {
            // bytes of BOTH CTAs land on this barrier
            const int kt_e = (C::BK == 128) ? 1 : ((kt & 1) == 0 ? 1 : 0);
            mbar_arrive_expect_tx(bar_full + 8 * s, 2 * (C::A_BYTES + C::B_BYTES + kt_e * C::E_BYTES));
          }
          tma_load_2d_pair(sbase + C::OFF_A + s * C::A_BYTES, &tmA, kt * (C::BK / 2), row0, full);
#pragma unroll
          for (int j = 0; j < C::B_SUBS; ++j)
            tma_load_2d_pair(sbase + C::OFF_B + s * C::B_BYTES + j * C::B_SUB_BYTES, &tmB,
                             kt * C::BK + j * 64, tok0, full);
          if (load_e) {
            const int kt128 = (C::BK == 128) ? kt : (kt >> 1);
            tma_load_1d_pair(sbase + C::OFF_E + s * C::E_BYTES, &tmE, (e_tile0 + kt128) * 256, full);
          }
          if (++s == C::STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (leader && elect_one()) {
      const uint32_t idesc = make_idesc_f16(256, C::BN, p.fmt, true);
      int s = 0;
      uint32_t ph = 0, aph = 0;
      uint32_t e_cols = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        ok = mbar_wait(bar_acce, aph ^ 1, err, p.status, 3);
        if (!ok) break;
        aph ^= 1;
        tc_fence_after();
        for (int kt = 0; kt < k_iters; ++kt) {
          ok = mbar_wait(bar_full + 8 * s, ph, err, p.status, 2);
          if (!ok) break;
          tc_fence_after();
          const bool new_e = (C::BK == 128) || ((kt & 1) == 0);
          if (new_e) {
            e_cols = C::E_COL0 + 4 * s;
            tc_cp_128x128b_pair(tmem_base + e_cols,
                                make_smem_desc(sbase + C::OFF_E + s * C::E_BYTES, 0, 128, kSwNone));
          }
          const uint32_t a_addr = sbase + C::OFF_A + s * C::A_BYTES;
          const uint32_t b_addr = sbase + C::OFF_B + s * C::B_BYTES;
#pragma unroll
          for (int kb = 0; kb < C::MMAS_PER_STAGE; ++kb) {
            const uint64_t adesc = (C::BK == 64)
                                       ? make_smem_desc(a_addr + kb * 32, 16, 512, kSw64)
                                       : make_smem_desc(a_addr + kb * 32, 16, 1024, kSw128);
            const uint64_t bdesc = make_smem_desc(
                b_addr + (kb >> 1) * C::B_SUB_BYTES + (kb & 1) * 64, 16, 1024, kSw128);
            const int ecol = (C::BK == 128) ? kb : ((kt & 1) * 2 + kb);
            tc_mma_sp_f16_pair(tmem_base, adesc, bdesc, tmem_base + e_cols + (ecol & ~1),
                               idesc | (ecol & 1), (kt > 0 || kb > 0) ? 1u : 0u);
          }
          tc_commit_pair(bar_empty + 8 * s);
          if (++s == C::STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        tc_commit_pair(bar_accf);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    const int q = warp & 3;                 // lane quadrant
    const int hf = (warp - 2) >> 2;         // which half of the token columns
    const uint32_t leader_acce = mapa_u32(bar_acce, 0);
    uint32_t aph = 0;
    bool ok = true;
    constexpr int NCH = C::COLS_PER_WARP / 32;        // 32-column chunks per warp
    constexpr int PK = (C::EPI == kEpiSwiGLU) ? 8 : 16;  // packed registers per chunk
    uint32_t packed[NCH * PK];
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
      const int m_blk = tile / p.num_n_blks;
      const int n_blk = tile % p.num_n_blks;
      {
        bool w = mbar_wait(bar_accf, aph, err, p.status, 4);
        ok = __all_sync(0xffffffffu, w);
      }
      if (!ok) break;
      aph ^= 1;
      tc_fence_after();
      const int row = m_blk * 256 + static_cast<int>(rank) * 128 + q * 32 + lane;  // weight row
      const int tok_w = n_blk * C::BN + hf * C::COLS_PER_WARP;                      // first token
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + hf * C::COLS_PER_WARP;
      float bias_v = 0.f;
      if (C::EPI == kEpiStore && p.bias != nullptr && row < p.n_out) bias_v = bias_at(p.bias, row, p.fmt);
      const bool upper = lane >= 16;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_acc + c * 32, r);
        tmem_ld_wait();
        if (C::EPI == kEpiStore) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float a = act_fn(__uint_as_float(r[2 * j]) + bias_v, p.act);
            const float b = act_fn(__uint_as_float(r[2 * j + 1]) + bias_v, p.act);
            packed[c * PK + j] = pack2(a, b, p.fmt);
          }
        } else {
          // lanes 0..15 hold gate(f), lanes 16..31 up(f); lower half-warp yields even tokens,
          // upper half-warp odd tokens of the chunk.
          float h[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const uint32_t send = upper ? r[2 * j] : r[2 * j + 1];
            const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 16);
            const float g = __uint_as_float(upper ? recv : r[2 * j]);
            const float u = __uint_as_float(upper ? r[2 * j + 1] : recv);
            const float sg = __fdividef(1.f, 1.f + __expf(-g));
            h[j] = (g * sg) * u;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) packed[c * PK + j] = pack2(h[2 * j], h[2 * j + 1], p.fmt);
        }
      }
      // accumulator fully drained: hand it back before touching global memory
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(leader_acce);

      uint16_t* y = static_cast<uint16_t*>(p.y);
      if (C::EPI == kEpiStore) {
        if (row < p.n_out) {
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = tok_w + c * 32 + 2 * j;
              const uint32_t v = packed[c * PK + j];
              if (t < p.m_tok) y[static_cast<size_t>(t) * p.ldy + row] = static_cast<uint16_t>(v & 0xFFFF);
              if (t + 1 < p.m_tok) y[static_cast<size_t>(t + 1) * p.ldy + row] = static_cast<uint16_t>(v >> 16);
            }
          }
        }
      } else {
        // feature index of this lane inside the hidden tensor
        const int f = (m_blk * 256 + static_cast<int>(rank) * 128 + q * 32) / 2 + (lane & 15);
        if (f < p.n_out / 2) {
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              // h index 2j, 2j+1 of this half-warp = tokens 4j + par and 4j + 2 + par of the chunk
              const int t = tok_w + c * 32 + 4 * j + (upper ? 1 : 0);
              const uint32_t v = packed[c * PK + j];
              if (t < p.m_tok) y[static_cast<size_t>(t) * p.ldy + f] = static_cast<uint16_t>(v & 0xFFFF);
              if (t + 2 < p.m_tok) y[static_cast<size_t>(t + 2) * p.ldy + f] = static_cast<uint16_t>(v >> 16);
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  if (*err) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer may still be signalling this CTA's barriers until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

template <class C>
int launch_pair_cfg(const SparseGemmArgs& a, cudaStream_t stream) {
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(sparse_gemm_pair_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::SMEM_BYTES) != cudaSuccess)
      return kErrCuda;
    attr_set[dev] = true;
  }
  CUtensorMap tmA, tmB, tmE;
  const uint64_t kc = static_cast<uint64_t>(a.K) / 2;
  if (!make_map_2d(&tmA, a.values, a.n_out, kc, kc * 2, 128, C::BK / 2,
                   C::BK == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, a.fmt))
    return kErrTensorMap;
  if (!make_map_2d(&tmB, a.x, a.m_tok, a.K, static_cast<uint64_t>(a.ldx) * 2, C::HALF_N, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B, a.fmt))
    return kErrTensorMap;
  if (!make_map_1d_u64(&tmE, a.meta, meta_bytes(a.n_out, a.K) / 8, 256)) return kErrTensorMap;
  PairParams p;
  p.bias = a.bias;
  p.y = a.y;
  p.status = a.status;
  p.n_out = a.n_out;
  p.m_tok = a.m_tok;
  p.K = a.K;
  p.ldy = a.ldy;
  p.num_m_blks = (a.n_out + 255) / 256;
  p.num_n_blks = (a.m_tok + C::BN - 1) / C::BN;
  p.k_tiles128 = (a.K + 127) / 128;
  p.fmt = a.fmt;
  p.act = a.act;
  const int tiles = p.num_m_blks * p.num_n_blks;
  int pairs = a.num_sms / 2;
  if (pairs > tiles) pairs = tiles;
  if (pairs < 1) pairs = 1;
  sparse_gemm_pair_kernel<C><<<2 * pairs, C::THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, tmE, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

}  // namespace

int launch_sparse_gemm_pair(const SparseGemmArgs& a, cudaStream_t stream) {
  if (a.K % 64 != 0 || a.K <= 0 || a.m_tok <= 0 || a.n_out <= 0) return kErrInvalid;
  if (a.n_out % 8 != 0 || a.ldx % 8 != 0) return kErrInvalid;
  if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.values) |
       reinterpret_cast<uintptr_t>(a.meta)) & 15)
    return kErrInvalid;
  const int variant = a.force_bn;  // 1256 / 1128: pair kernel with BN 256 / 128
  if (a.epi == kEpiSwiGLU) {
    if (a.n_out % 32 != 0) return kErrInvalid;
    if (variant == 1128) return launch_pair_cfg<PairCfg<128, 128, 4, kEpiSwiGLU>>(a, stream);
    return launch_pair_cfg<PairCfg<256, 128, 4, kEpiSwiGLU>>(a, stream);
  }
  if (variant == 1128) return launch_pair_cfg<PairCfg<128, 128, 4, kEpiStore>>(a, stream);
  return launch_pair_cfg<PairCfg<256, 128, 4, kEpiStore>>(a, stream);
}

}  // namespace sfb200
