// 2:4-sparse GEMM for sm_100a, split-K over a thread-block cluster: the variant for token counts
// between decode and prefill when the weight has too few 128-row tiles to fill the GPU (a
// 4096-row down or attention projection has 32, the B200 has 148 SMs).
//
// Same operand formats, tensor-memory layout and call sites as sparse_gemm_sm100.cu.  A cluster of
// S CTAs (S = 2 or 4) owns one 128-row x BN-token output tile; CTA r of the cluster streams the
// r-th slice of K through the same TMA -> tcgen05.mma.sp pipeline, so the weight is read from HBM
// by S times as many SMs.  The partial accumulators are reduced through distributed shared
// memory, with no scratch in global memory and no atomics:
//   1. every CTA drains its fp32 accumulator from tensor memory and stores feature block o
//      (128/S features) into a slot of CTA o's shared memory (st.shared::cluster);
//   2. one cluster barrier;
//   3. CTA o sums its S slots in rank order (fixed order: results do not depend on timing), adds
//      the bias, applies the activation and writes the 16-bit outputs.
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

struct SplitKParams {
  const uint32_t* meta;   // [row_tiles][k_tiles][128][4]
  const void* bias;       // per out feature, 16-bit type, or null
  void* y;                // [m_tok, n_out], row pitch ldy elements
  int* status;            // device status word
  int n_out, m_tok, K, ldy;
  int k_tiles128;         // ceil(K / 128): metadata tiles along K
  int num_n_blks;         // ceil(m_tok / BN)
  int split;              // S: CTAs per cluster = K slices
  int fmt, act;
};

// One pipeline stage = one 128-wide K tile = one metadata tile.  (With 64-wide stages the K loop ran at
// one stage per ~160-190 ns whatever the tile held: the per-stage handshake, not the bytes, set the
// pace, so stages are made as wide as the 128-byte swizzle of the A operand allows.)
template <int BN_, int STAGES_>
struct SkCfg {
  static constexpr int BM = 128, BK = 128;
  static constexpr int BN = BN_, STAGES = STAGES_;
  static constexpr int A_BYTES = BM * (BK / 2) * 2;   // 16 KiB, 128-byte swizzle
  static constexpr int B_SUB_BYTES = BN * 128;        // BN tokens x 64 elements
  static constexpr int B_BYTES = 2 * B_SUB_BYTES;
  static constexpr int E_BYTES = 2048;                // one 128 x 128 metadata tile per stage
  static constexpr int SLOT_BYTES = BN * BM * 4;      // S slots x BN tokens x 128/S features, fp32
  static constexpr int TMEM_USED = BN + 4 * STAGES;
  static constexpr int TMEM_COLS = TMEM_USED <= 64 ? 64 : TMEM_USED <= 128 ? 128 : TMEM_USED <= 256 ? 256 : 512;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_E = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_SLOT = OFF_E + STAGES * E_BYTES;
  static constexpr int OFF_BAR = OFF_SLOT + SLOT_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 128, "BN");
  static_assert(8 * (2 * STAGES + 1) + 16 <= 256, "barrier area");
  static_assert(SMEM_BYTES <= 232448, "smem");
};

__device__ __forceinline__ float sk_act(float v, int act) {
  switch (act) {
    case kActRelu: return fmaxf(v, 0.f);
    case kActSilu: return v * __fdividef(1.f, 1.f + __expf(-v));
    case kActGelu: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    default: return v;
  }
}

template <class C>
__global__ void __launch_bounds__(192, 1)
sparse_gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const SplitKParams p) {
  extern __shared__ uint8_t smem_raw[];
  // the same offset in every CTA of the cluster: the dynamic shared memory base is identical
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * C::STAGES;
  const uint32_t bar_accf = bar_empty + 8 * C::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + 8 * (2 * C::STAGES + 1));
  volatile int* err = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = p.split;
  const int rank = static_cast<int>(cluster_ctarank());
  const int tile = blockIdx.x / S;
  const int m_blk = tile / p.num_n_blks;
  const int n_blk = tile % p.num_n_blks;
  // K slice of this CTA, in 128-wide metadata tiles, then in 64-wide pipeline stages
  const int base = p.k_tiles128 / S, extra = p.k_tiles128 % S;
  const int t_begin = rank * base + (rank < extra ? rank : extra);
  const int t_count = base + (rank < extra ? 1 : 0);
  const int kt_begin = t_begin;              // stages are whole metadata tiles; a trailing half tile (K % 128 == 64)
  const int kt_end = t_begin + t_count;      // is zero-filled by TMA

  if (threadIdx.x == 0) {
    *err = 0;
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_accf, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // First cluster barrier, split: arrive now, wait only before the first store into a peer's slots
  // (its purpose is that every CTA of the cluster is resident by then), so the K loop does not pay for it.
  cluster_arrive();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      for (int kt = kt_begin; kt < kt_end; ++kt) {
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, err, p.status, 1)) break;
        const uint32_t full = bar_full + 8 * s;
        mbar_arrive_expect_tx(full, C::A_BYTES + C::B_BYTES + C::E_BYTES);
        tma_load_2d(sbase + C::OFF_A + s * C::A_BYTES, &tmA, kt * (C::BK / 2), m_blk * C::BM, full);
        tma_load_2d(sbase + C::OFF_B + s * C::B_BYTES, &tmB, kt * C::BK, n_blk * C::BN, full);
        tma_load_2d(sbase + C::OFF_B + s * C::B_BYTES + C::B_SUB_BYTES, &tmB, kt * C::BK + 64, n_blk * C::BN, full);
        const uint32_t* src = p.meta + (static_cast<size_t>(m_blk) * p.k_tiles128 + kt) * 512;
        bulk_load_1d(sbase + C::OFF_E + s * C::E_BYTES, src, C::E_BYTES, full);
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_f16(C::BM, C::BN, p.fmt, true);
      int s = 0;
      uint32_t ph = 0;
      uint32_t e_cols = 0;
      bool ok = true;
      for (int kt = kt_begin; kt < kt_end; ++kt) {
        ok = mbar_wait(bar_full + 8 * s, ph, err, p.status, 2);
        if (!ok) break;
        tc_fence_after();
        e_cols = C::BN + 4 * s;
        tc_cp_128x128b(tmem_base + e_cols, make_smem_desc(sbase + C::OFF_E + s * C::E_BYTES, 0, 128, kSwNone));
        const uint32_t a_addr = sbase + C::OFF_A + s * C::A_BYTES;
        const uint32_t b_addr = sbase + C::OFF_B + s * C::B_BYTES;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          const uint64_t adesc = make_smem_desc(a_addr + kb * 32, 16, 1024, kSw128);
          const uint64_t bdesc = make_smem_desc(b_addr + (kb >> 1) * C::B_SUB_BYTES + (kb & 1) * 64, 16, 1024, kSw128);
          tc_mma_sp_f16(tmem_base, adesc, bdesc, tmem_base + e_cols + (kb & ~1), idesc | (kb & 1),
                        (kt > kt_begin || kb > 0) ? 1u : 0u);
        }
        tc_commit(bar_empty + 8 * s);
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
      }
      if (ok) tc_commit(bar_accf);
    }
  } else {
    // ------------------------------------------------------------ drain: partial tile -> owners' slots
    const int q = warp & 3;                    // tensor-memory lane quadrant = features q*32 .. q*32+31
    const int fpo = C::BM / S;                 // features per owner
    const int owner = (q * 32) / fpo;
    const int f_in_owner = (q * 32) % fpo + lane;
    int n_chunks = C::BN / 32;
    {
      const int need = (p.m_tok - n_blk * C::BN + 31) / 32;
      if (need < n_chunks) n_chunks = need;
    }
    const bool have = kt_end > kt_begin;
    bool ok = true;
    if (have) ok = mbar_wait(bar_accf, 0, err, p.status, 4);
    __syncwarp();
    cluster_wait();
    if (ok) {
      tc_fence_after();
      // slot[src rank][token][feature in owner], fp32
      const uint32_t slot0 = mapa_u32(sbase + C::OFF_SLOT, owner) +
                             static_cast<uint32_t>((rank * C::BN * fpo + f_in_owner) * 4);
      uint32_t r[32];
      for (int c = 0; c < n_chunks; ++c) {
        if (have) {
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j)
          st_cluster_f32(slot0 + static_cast<uint32_t>((c * 32 + j) * fpo * 4), __uint_as_float(r[j]));
      }
    }
  }

  __syncwarp();
  if (warp < 2) cluster_wait();   // producer and MMA warps: second half of the first barrier
  tc_fence_before();
  cluster_sync_all();   // all partials have landed in their owners' shared memory

  if (warp >= 2 && *err == 0) {
    // ------------------------------------------------------------ reduce own feature block, write out
    const int fpo = C::BM / S;
    const float* slots = reinterpret_cast<const float*>(smem + C::OFF_SLOT);
    const int tok_base = n_blk * C::BN;
    int n_tok = p.m_tok - tok_base;
    if (n_tok > C::BN) n_tok = C::BN;
    const int feat0 = m_blk * C::BM + rank * fpo;
    uint16_t* y = static_cast<uint16_t*>(p.y);
    const uint16_t* bias = static_cast<const uint16_t*>(p.bias);
    for (int f = lane; f < fpo; f += 32) {
      const int feat = feat0 + f;
      if (feat >= p.n_out) break;
      float bv = 0.f;
      if (bias != nullptr)
        bv = p.fmt == 1 ? __bfloat162float(__ushort_as_bfloat16(bias[feat])) : __half2float(__ushort_as_half(bias[feat]));
      for (int t = warp - 2; t < n_tok; t += 4) {
        float v = 0.f;
        for (int src = 0; src < S; ++src) v += slots[(src * C::BN + t) * fpo + f];
        v = sk_act(v + bv, p.act);
        const uint16_t b = p.fmt == 1 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
        y[static_cast<size_t>(tok_base + t) * p.ldy + feat] = b;
      }
    }
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  if (*err) {
    // give copies that may still be in flight time to land before shared memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <class C>
int launch_sk(const SparseGemmArgs& a, int split, cudaStream_t stream) {
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(sparse_gemm_splitk_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::SMEM_BYTES) != cudaSuccess)
      return kErrCuda;
    attr_set[dev] = true;
  }
  CUtensorMap tmA, tmB;
  const uint64_t kc = static_cast<uint64_t>(a.K) / 2;
  if (!make_map_2d(&tmA, a.values, a.n_out, kc, kc * 2, C::BM, C::BK / 2, CU_TENSOR_MAP_SWIZZLE_128B, a.fmt))
    return kErrTensorMap;
  if (!make_map_2d(&tmB, a.x, a.m_tok, a.K, static_cast<uint64_t>(a.ldx) * 2, C::BN, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B, a.fmt))
    return kErrTensorMap;
  SplitKParams p;
  p.meta = static_cast<const uint32_t*>(a.meta);
  p.bias = a.bias;
  p.y = a.y;
  p.status = a.status;
  p.n_out = a.n_out;
  p.m_tok = a.m_tok;
  p.K = a.K;
  p.ldy = a.ldy;
  p.k_tiles128 = (a.K + 127) / 128;
  p.num_n_blks = (a.m_tok + C::BN - 1) / C::BN;
  p.split = split;
  p.fmt = a.fmt;
  p.act = a.act;
  const int tiles = ((a.n_out + C::BM - 1) / C::BM) * p.num_n_blks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * split), 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(split);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, sparse_gemm_splitk_kernel<C>, tmA, tmB, p) != cudaSuccess) {
    cudaGetLastError();
    return kErrCuda;
  }
  return kOk;
}

}  // namespace

int splitk_token_tile(int m_tok) { return m_tok <= 32 ? 32 : m_tok <= 64 ? 64 : 128; }

int splitk_factor(int m_tok, int n_out, int K, int num_sms) {
  const int bn = splitk_token_tile(m_tok);
  const int tiles = ((n_out + 127) / 128) * ((m_tok + bn - 1) / bn);
  const int k128 = (K + 127) / 128;
  int s = 1;
  if (tiles * 4 <= num_sms) s = 4;
  else if (tiles * 2 <= num_sms) s = 2;
  while (s > 1 && k128 < 4 * s) s >>= 1;   // at least four metadata tiles (K = 512) per slice
  if (bn == 128 && s == 2) s = 1;          // measured: two slices of a 128-token tile gain nothing (X traffic dominates)
  return s;
}

int launch_sparse_gemm_splitk(const SparseGemmArgs& a, int split, cudaStream_t stream) {
  if (a.K % 64 != 0 || a.K <= 0 || a.m_tok <= 0 || a.n_out <= 0) return kErrInvalid;
  if (a.n_out % 8 != 0 || a.ldx % 8 != 0) return kErrInvalid;
  if (a.epi != kEpiStore) return kErrInvalid;
  if (split != 2 && split != 4) return kErrInvalid;
  if ((a.K + 127) / 128 < split) return kErrInvalid;
  if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.values) |
       reinterpret_cast<uintptr_t>(a.meta)) & 15)
    return kErrInvalid;
  int bn = a.force_bn >= 3000 ? a.force_bn % 1000 : splitk_token_tile(a.m_tok);
  switch (bn) {
    case 32: return launch_sk<SkCfg<32, 7>>(a, split, stream);
    case 64: return launch_sk<SkCfg<64, 5>>(a, split, stream);
    case 128: return launch_sk<SkCfg<128, 3>>(a, split, stream);
    default: return kErrInvalid;
  }
}

}  // namespace sfb200
