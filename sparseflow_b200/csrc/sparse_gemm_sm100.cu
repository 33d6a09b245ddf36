// 2:4-sparse GEMM for sm_100a:  Y[tokens, out] = X[tokens, K] . W[out, K]^T  with W held as
// compressed values [out, K/2] + tiled 2-bit metadata (layout: see prune_compress.cu).
//
// Replaces the reference's sparse matmul call sites (sparseflow/fused_mlp.py:54,60,
// sparseflow/nn/sparseflow_linear.py:123, sparseflow/nn/sparseflow_mlp.py:95,97), which go to
// PyTorch's Ampere semi-structured kernels, and the fused SiLU.mul of
// sparseflow/kernels/fused_silu_mul.py:6-31 (here an epilogue of the gate|up GEMM).
//
// Mapping onto tcgen05.mma.sp (kind::f16, fp32 accumulate in tensor memory):
//   MMA A operand (sparse, M=128 rows)  = 128 weight rows, K-major compressed values in smem
//   MMA B operand (dense,  N=BN rows)   = BN tokens of X, K-major in smem
//   MMA D (128 lanes x BN columns fp32) = Y^T tile: lane = out feature, column = token
//   metadata: 128 lanes x 1 column per K=32 instruction, copied smem -> tmem with tcgen05.cp
//
// One persistent CTA per SM, 6 warps: warp 0 = TMA producer, warp 1 = MMA issuer (one thread) and
// tensor-memory owner, warps 2..5 = epilogue (tmem -> registers -> smem -> TMA store).
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

struct GemmParams {
  const uint32_t* meta;   // [row_tiles][k_tiles][128][4]
  const void* bias;       // per out feature, 16-bit type, or null
  int* status;            // device status word
  int n_out;              // weight rows
  int m_tok;              // tokens
  int K;                  // logical K
  int k_tiles128;         // ceil(K / 128): metadata tiles along K
  int num_m_blks;         // ceil(n_out / 128)
  int num_n_blks;         // ceil(m_tok / BN)
  int fmt;                // 0 = f16, 1 = bf16
  int act;                // Activation for EPI_STORE
};

template <int BN_, int BK_, int STAGES_, int EPI_>
struct Cfg {
  static constexpr int BM = 128;
  static constexpr int BN = BN_;
  static constexpr int BK = BK_;
  static constexpr int STAGES = STAGES_;
  static constexpr int EPI = EPI_;
  static constexpr int A_BYTES = BM * (BK / 2) * 2;
  static constexpr int B_SUBS = BK / 64;          // 64-element (128 B) wide sub tiles of X
  static constexpr int B_SUB_BYTES = BN * 128;
  static constexpr int B_BYTES = B_SUBS * B_SUB_BYTES;
  static constexpr int E_BYTES = 2048;            // one 128x128 metadata tile
  static constexpr int MMAS_PER_STAGE = BK / 32;
  static constexpr int ACC_STAGES = (2 * BN + 4 * STAGES <= 512) ? 2 : 1;
  static constexpr int TMEM_USED = ACC_STAGES * BN + 4 * STAGES;
  static constexpr int TMEM_COLS = TMEM_USED <= 32 ? 32 : TMEM_USED <= 64 ? 64 : TMEM_USED <= 128 ? 128
                                   : TMEM_USED <= 256 ? 256 : 512;
  static constexpr int D_ROWS = 32;               // tokens per store chunk
  static constexpr int D_COLS = (EPI == kEpiSwiGLU) ? 64 : 128;
  static constexpr int D_BYTES = D_ROWS * D_COLS * 2;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_E = OFF_B + STAGES * B_BYTES;
  static constexpr int OFF_D = OFF_E + STAGES * E_BYTES;
  static constexpr int OFF_BAR = OFF_D + 2 * D_BYTES;
  static constexpr int BAR_BYTES = ((8 * (2 * STAGES + 4) + 16) + 127) & ~127;   // barriers + tmem slot + error flag
  static constexpr int SMEM_BYTES = OFF_BAR + BAR_BYTES + 1024;  // + alignment slack
  static_assert(BK == 64 || BK == 128, "BK");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "BN");
  static_assert(TMEM_USED <= 512, "tmem");
  static_assert(SMEM_BYTES <= 232448, "smem");
};

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case kActRelu: return fmaxf(v, 0.f);
    case kActSilu: return v * __fdividef(1.f, 1.f + __expf(-v));
    case kActGelu: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    default: return v;
  }
}

__device__ __forceinline__ uint16_t to_bits16(float v, int fmt) {
  if (fmt == 1) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  return __half_as_ushort(__float2half_rn(v));
}
__device__ __forceinline__ float from_bits16(uint16_t b, int fmt) {
  if (fmt == 1) return __bfloat162float(__ushort_as_bfloat16(b));
  return __half2float(__ushort_as_half(b));
}

template <class C>
__global__ void __launch_bounds__(192, 1)
sparse_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmD, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  // barrier slots: full[S], empty[S], acc_full[2], acc_empty[2]
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * C::STAGES;
  const uint32_t bar_accf = bar_empty + 8 * C::STAGES;
  const uint32_t bar_acce = bar_accf + 8 * 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + 8 * (2 * C::STAGES + 4));
  volatile int* err = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_blks * p.num_n_blks;
  const int k_iters = (p.K + C::BK - 1) / C::BK;

  if (threadIdx.x == 0) {
    *err = 0;
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_accf + 8 * a, 1);
      mbar_init(bar_acce + 8 * a, 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile / p.num_n_blks;
        const int n_blk = tile % p.num_n_blks;
        for (int kt = 0; kt < k_iters; ++kt) {
          ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, err, p.status, 1);
          if (!ok) break;
          const bool load_e = (C::BK == 128) || ((kt & 1) == 0);
          const uint32_t full = bar_full + 8 * s;
          mbar_arrive_expect_tx(full, C::A_BYTES + C::B_BYTES + (load_e ? C::E_BYTES : 0));
          tma_load_2d(sbase + C::OFF_A + s * C::A_BYTES, &tmA, kt * (C::BK / 2), m_blk * C::BM, full);
#pragma unroll
          for (int j = 0; j < C::B_SUBS; ++j)
            tma_load_2d(sbase + C::OFF_B + s * C::B_BYTES + j * C::B_SUB_BYTES, &tmB,
                        kt * C::BK + j * 64, n_blk * C::BN, full);
          if (load_e) {
            const int kt128 = (C::BK == 128) ? kt : (kt >> 1);
            const uint32_t* src =
                p.meta + (static_cast<size_t>(m_blk) * p.k_tiles128 + kt128) * 512;
            bulk_load_1d(sbase + C::OFF_E + s * C::E_BYTES, src, C::E_BYTES, full);
          }
          if (++s == C::STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_f16(C::BM, C::BN, p.fmt, true);
      int s = 0;
      uint32_t ph = 0;
      int as = 0;
      uint32_t aph = 0;
      uint32_t e_cols = 0;  // tmem column base of the metadata tile in use
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        ok = mbar_wait(bar_acce + 8 * as, aph ^ 1, err, p.status, 3);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * C::BN;
        for (int kt = 0; kt < k_iters; ++kt) {
          ok = mbar_wait(bar_full + 8 * s, ph, err, p.status, 2);
          if (!ok) break;
          tc_fence_after();
          const bool new_e = (C::BK == 128) || ((kt & 1) == 0);
          if (new_e) {
            e_cols = C::ACC_STAGES * C::BN + 4 * s;
            const uint64_t edesc =
                make_smem_desc(sbase + C::OFF_E + s * C::E_BYTES, 0, 128, kSwNone);
            tc_cp_128x128b(tmem_base + e_cols, edesc);
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
            tc_mma_sp_f16(d_tmem, adesc, bdesc, tmem_base + e_cols + (ecol & ~1),
                          idesc | (ecol & 1), (kt > 0 || kb > 0) ? 1u : 0u);
          }
          tc_commit(bar_empty + 8 * s);
          if (++s == C::STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        tc_commit(bar_accf + 8 * as);
        if (++as == C::ACC_STAGES) { as = 0; aph ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                       // tensor-memory lane quadrant of this warp
    const bool store_thread = (threadIdx.x == 64);
    int as = 0;
    uint32_t aph = 0;
    uint32_t chunk_ctr = 0;
    bool ok = true;
    uint32_t r[32];
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m_blk = tile / p.num_n_blks;
      const int n_blk = tile % p.num_n_blks;
      ok = mbar_wait(bar_accf + 8 * as, aph, err, p.status, 4);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * C::BN;
      const int tok_base = n_blk * C::BN;
      int n_chunks = C::BN / 32;
      {
        const int rem = p.m_tok - tok_base;
        const int need = (rem + 31) / 32;
        if (need < n_chunks) n_chunks = need;
      }
      float bias_v = 0.f;
      if (C::EPI == kEpiStore && p.bias != nullptr) {
        const int o = m_blk * C::BM + q * 32 + lane;
        if (o < p.n_out) bias_v = from_bits16(static_cast<const uint16_t*>(p.bias)[o], p.fmt);
      }
      for (int c = 0; c < n_chunks; ++c) {
        tmem_ld_32x32(t_acc + c * 32, r);
        tmem_ld_wait();
        if (c == n_chunks - 1) {
          // accumulator fully read: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acce + 8 * as);
        }
        const uint32_t db = chunk_ctr & 1;
        ++chunk_ctr;
        uint8_t* stage = smem + C::OFF_D + db * C::D_BYTES;
        if (store_thread) tma_store_wait_read<1>();
        named_bar_sync(1, 128);
        if (C::EPI == kEpiStore) {
          uint16_t* srow = reinterpret_cast<uint16_t*>(stage) + q * 32 + lane;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float v = __uint_as_float(r[j]) + bias_v;
            v = apply_act(v, p.act);
            srow[j * C::D_COLS] = to_bits16(v, p.fmt);
          }
        } else {
          // rows come in blocks of 16 gate rows then the 16 matching up rows: lanes 0..15 hold
          // gate(f), lanes 16..31 hold up(f).  Per token pair, the lower half-warp produces token
          // j, the upper half-warp token j+1.
          const bool upper = lane >= 16;
          uint16_t* scol = reinterpret_cast<uint16_t*>(stage) + q * 16 + (lane & 15);
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const uint32_t send = upper ? r[j] : r[j + 1];
            const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 16);
            const float g = __uint_as_float(upper ? recv : r[j]);
            const float u = __uint_as_float(upper ? r[j + 1] : recv);
            const float sgm = __fdividef(1.f, 1.f + __expf(-g));
            const float h = (g * sgm) * u;
            scol[(j + (upper ? 1 : 0)) * C::D_COLS] = to_bits16(h, p.fmt);
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (store_thread) {
          tma_store_2d(&tmD, smem_u32(stage), m_blk * C::D_COLS, tok_base + c * 32);
          tma_store_commit();
        }
      }
      if (++as == C::ACC_STAGES) { as = 0; aph ^= 1; }
    }
    if (store_thread) tma_store_wait_all<0>();
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

// ------------------------------------------------------------------ host side
template <class C>
int launch_cfg(const SparseGemmArgs& a, cudaStream_t stream) {
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(sparse_gemm_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             C::SMEM_BYTES) != cudaSuccess)
      return kErrCuda;
    attr_set[dev] = true;
  }
  CUtensorMap tmA, tmB, tmD;
  const uint64_t kc = static_cast<uint64_t>(a.K) / 2;
  if (!make_map_2d(&tmA, a.values, a.n_out, kc, kc * 2, C::BM, C::BK / 2,
                   C::BK == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, a.fmt))
    return kErrTensorMap;
  if (!make_map_2d(&tmB, a.x, a.m_tok, a.K, static_cast<uint64_t>(a.ldx) * 2, C::BN, 64,
                   CU_TENSOR_MAP_SWIZZLE_128B, a.fmt))
    return kErrTensorMap;
  const int out_cols = (C::EPI == kEpiSwiGLU) ? a.n_out / 2 : a.n_out;
  if (!make_map_2d(&tmD, a.y, a.m_tok, out_cols, static_cast<uint64_t>(a.ldy) * 2, C::D_ROWS,
                   C::D_COLS, CU_TENSOR_MAP_SWIZZLE_NONE, a.fmt))
    return kErrTensorMap;
  GemmParams p;
  p.meta = static_cast<const uint32_t*>(a.meta);
  p.bias = a.bias;
  p.status = a.status;
  p.n_out = a.n_out;
  p.m_tok = a.m_tok;
  p.K = a.K;
  p.k_tiles128 = (a.K + 127) / 128;
  p.num_m_blks = (a.n_out + C::BM - 1) / C::BM;
  p.num_n_blks = (a.m_tok + C::BN - 1) / C::BN;
  p.fmt = a.fmt;
  p.act = a.act;
  const int tiles = p.num_m_blks * p.num_n_blks;
  int grid = a.num_sms < tiles ? a.num_sms : tiles;
  if (grid < 1) grid = 1;
  sparse_gemm_kernel<C><<<grid, 192, C::SMEM_BYTES, stream>>>(tmA, tmB, tmD, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

// Kernel / token-tile choice from 129 tokens up: the cheapest, by estimated time, of the single-CTA tiles and the
// CTA-pair tiles.  Up to about a thousand tokens every candidate is bound by operand traffic, not by the tensor pipe,
// and what decides is how many passes ("waves") the tile count needs on the available SMs (or SM pairs):
//   single-CTA tile of bn tokens: waves x 64-wide K steps x step time + 8.5 us, where a step moves 9 KiB (values +
//     metadata) + bn x 128 B (tokens), an SM sustains about 145 GB/s of operand traffic and all SMs together about
//     19.5 TB/s out of L2 (17 TB/s for the 256-token tile, whose ring is only four stages deep);
//   CTA-pair tiles: pick_pair_variant's estimate.
// Measured on B200 (variants timed as CUDA graphs against this model): 22016 x 4096 at 1024 tokens 112 -> 88 us with the
// 256 x 208 pair tile; 4096 x 11008 at 1024 tokens stays with the single-CTA 256-token tile (32 row tiles x 4 = 128 tiles
// = one wave on 148 SMs, 59.6 us, against two waves of pair tiles, 66 us).
int pick_mid_variant(int n_out, int m_tok, int K, int num_sms, int swiglu) {
  const double k64 = (K + 63) / 64;
  const long mb = (n_out + 127) / 128;
  double best = 1e30;
  int pick = 128;
  const int cands[3] = {128, 192, 256};   // a 64-token tile costs the same per step (latency-bound ring): measured no gain
  for (int bn : cands) {
    const long tiles = mb * ((m_tok + bn - 1) / bn);
    const long waves = (tiles + num_sms - 1) / num_sms;
    const double active = tiles < num_sms ? static_cast<double>(tiles) : static_cast<double>(num_sms);
    const double bytes = 9216.0 + bn * 128.0;
    const double per_sm = bytes / 145e9, shared = active * bytes / (bn == 256 ? 17e12 : 19.5e12);
    const double cost = (waves * k64 * (per_sm > shared ? per_sm : shared) + 8.5e-6) * 1e6;
    if (cost < best) { best = cost; pick = bn; }
  }
  double pcost = 1e30;
  const int pv = pick_pair_variant(n_out, m_tok, K, num_sms, swiglu, &pcost);
  if (pcost < 0.97 * best) pick = pv;
  return pick;
}

template <int EPI>
int dispatch_bn(const SparseGemmArgs& a, cudaStream_t stream) {
  const int bn = a.force_bn;
  switch (bn) {
    // 128-wide stages: the per-stage handshake (~160-190 ns), not the bytes, paces the K loop of the small tiles
    case 32: return launch_cfg<Cfg<32, 128, 7, EPI>>(a, stream);
    case 64: return launch_cfg<Cfg<64, 128, 6, EPI>>(a, stream);
    case 128: return launch_cfg<Cfg<128, 128, 4, EPI>>(a, stream);
    case 192: return launch_cfg<Cfg<192, 64, 6, EPI>>(a, stream);
    case 256: return launch_cfg<Cfg<256, 64, 4, EPI>>(a, stream);
    default: return kErrInvalid;
  }
}

}  // namespace

int plan_sparse_gemm(int m_tok, int n_out, int K, int epi, int num_sms) {
  // few row tiles (the weight has fewer 128-row tiles than half the SMs) and fewer tokens than the
  // prefill kernel wants: split K over a cluster so that the weight is streamed by (nearly) every SM
  const int split = (epi == kEpiStore && m_tok < kPairMinTokens) ? splitk_factor(m_tok, n_out, K, num_sms) : 1;
  // decode-sized token counts: bandwidth kernel on warp-level mma.sp; measured against the split-K
  // kernel it only wins at 1-2 tokens when both apply
  if (m_tok <= kSmallMMaxTokens && (split == 1 || m_tok <= 2)) return 8;
  if (m_tok >= 4 * kPairMinTokens) return pick_pair_variant(n_out, m_tok, K, num_sms, epi == kEpiSwiGLU);   // prefill proper: pair tiles
  if (m_tok > 64 && m_tok <= 128) {
    // 65..128 tokens: one 128-token tile per row tile, two 64-token tiles, or split K.  A 128-wide stage of the
    // 128-token tile holds 50 KB and is feed-bound (~430 ns), of the 64-token tile 34 KB (~268 ns); what decides is
    // again the number of passes over the SMs.  (Measured: 8192 x 8192 at 128 tokens 27.9 -> 20.5 us with two
    // 64-token tiles; 22016 x 4096 31.6 -> 28.9 us; 11008 x 4096 and 28672 x 4096 stay with the 128-token tile.)
    const long mb = (n_out + 127) / 128;
    const double k128 = (K + 127) / 128;
    auto waves = [&](long tiles) { return static_cast<double>((tiles + num_sms - 1) / num_sms); };
    const double c128 = waves(mb) * k128 * 430e-9 + 4e-6;
    const double c64 = waves(2 * mb) * k128 * 268e-9 + 4e-6;
    const double csplit = split > 1 ? (k128 / split) * 385e-9 + 10e-6 : 1e30;
    if (epi == kEpiStore && csplit < c128 && csplit < c64) return (split == 4 ? 4000 : 3000) + 128;
    return c64 < c128 ? 64 : 128;
  }
  if (split > 1) return (split == 4 ? 4000 : 3000) + splitk_token_tile(m_tok);
  if (m_tok <= 32) return 32;
  if (m_tok <= 64) return 64;
  return pick_mid_variant(n_out, m_tok, K, num_sms, epi == kEpiSwiGLU);
}

int launch_sparse_gemm(const SparseGemmArgs& a, cudaStream_t stream) {
  if (a.K % 64 != 0 || a.K <= 0 || a.m_tok <= 0 || a.n_out <= 0) return kErrInvalid;
  if (a.n_out % 8 != 0 || a.ldx % 8 != 0 || a.ldy % 8 != 0) return kErrInvalid;
  if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.values) |
       reinterpret_cast<uintptr_t>(a.meta) | reinterpret_cast<uintptr_t>(a.y)) & 15)
    return kErrInvalid;
  if (a.epi == kEpiSwiGLU && (a.n_out % 32 != 0 || (a.n_out / 2) % 8 != 0)) return kErrInvalid;
  SparseGemmArgs b = a;
  if (a.out_f32) {
    // fp32 output exists in the CTA-pair kernel's epilogue only
    if (a.epi != kEpiStore) return kErrInvalid;
    if (b.force_bn < 1000 || (b.force_bn >= 3000 && b.force_bn < 5000))
      b.force_bn = pick_pair_variant(a.n_out, a.m_tok, a.K, a.num_sms, 0);
    return launch_sparse_gemm_pair(b, stream);
  }
  if (b.force_bn == 0) b.force_bn = plan_sparse_gemm(a.m_tok, a.n_out, a.K, a.epi, a.num_sms);
  const int v = b.force_bn;
  if (v == 8) return launch_sparse_gemm_small_m(b, stream);
  if (v >= 5000) return launch_sparse_gemm_pair(b, stream);
  if (v >= 3000) return launch_sparse_gemm_splitk(b, v >= 4000 ? 4 : 2, stream);
  if (v >= 1000) return launch_sparse_gemm_pair(b, stream);
  return a.epi == kEpiSwiGLU ? dispatch_bn<kEpiSwiGLU>(b, stream) : dispatch_bn<kEpiStore>(b, stream);
}

}  // namespace sfb200
