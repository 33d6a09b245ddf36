// Small-M (decode) 2:4-sparse GEMM:  Y[M, N] = act(X[M, K] . W^T + bias),  M <= 32 tokens.
//
// The reference has no sparse path here (its gate sends M < 32 to dense,
// sparseflow/dispatch.py:40).  At these token counts the GEMM is bound by streaming the weight
// from HBM once, and the compressed weight is 0.5625x the dense bytes (values K/2*2 B + metadata
// K/8 B per row), so this kernel is built for bandwidth, on warp-level primitives:
//   * a work unit is SL slabs of 16 weight rows over the full K (SL = 2 for the fused gate|up
//     weight: its rows come as 16 gate rows then the 16 matching up rows, so one unit yields 16
//     finished hidden features and SiLU.mul is applied in the reduction, with no scratch buffer);
//     persistent CTAs (a multiple of the SM count) walk the units; the 8 warps of a CTA split K
//     and reduce through shared memory;
//   * each warp streams its 16 x K/8 slice of compressed values with a 4-deep cp.async ring
//     (16-byte copies, 128 B contiguous per row and stage), reads fragments with ldmatrix, and
//     multiplies with mma.sp m16n8k32 (fp32 accumulate), one instruction per 8 tokens;
//   * metadata needs no decoding: the 32-bit words of the tiled layout ([row m | row m+8] x 16
//     logical K) are exactly what mma.sp takes from lanes 4g and 4g+1;
//   * metadata needs no decoding either way it arrives: the slab's 256 B per K tile ride the same
//     cp.async ring as the values, so no MMA waits on a DRAM-latency load;
//   * X is tiny and every slab re-reads the same K slice per warp: each warp keeps its slice in
//     shared memory already in B-fragment order (one 16-byte read per k-step and 8 tokens) when it
//     fits, else reads it through L1.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace sfb200 {
namespace {

constexpr int kWarps = 8;
__host__ __device__ constexpr int kStagesFor(int sl) { return sl == 1 ? 4 : 4; }   // ring depth (deeper rings measured no faster)
constexpr int kRowPitch = 144;                        // 128 B of values + 16 B pad: conflict-free ldmatrix
constexpr int kValBytes = 16 * kRowPitch;             // one 16-row x 128-logical-K chunk of values
constexpr int kStageBytes = kValBytes + 256;          // + the slab's metadata for that K tile (16 lanes x 16 B)
__host__ __device__ constexpr int kWarpSmemFor(int sl) { return kStagesFor(sl) * sl * kStageBytes; }
constexpr int kMaxNT = 4;                             // up to 32 tokens

struct SmallParams {
  const uint16_t* x;
  const uint16_t* values;
  const uint32_t* meta;
  const uint16_t* bias;
  uint16_t* y;
  int m_tok, n_out, K, ldx, ldy;
  int k_tiles128;
  int num_slabs;
  int fmt, act;
  int xs_ksteps;   // > 0: per-warp shared-memory cache of X fragments, this many 32-wide k-steps per warp
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma_sp_16832(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[4],
                                             uint32_t e) {
  if (BF16) {
    asm volatile(
        "mma.sp::ordered_metadata.sync.aligned.m16n8k32.row.col.f32.bf16.bf16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(e));
  } else {
    asm volatile(
        "mma.sp::ordered_metadata.sync.aligned.m16n8k32.row.col.f32.f16.f16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9, %10, %11}, {%0, %1, %2, %3}, %12, 0x0;"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(e));
  }
}
__device__ __forceinline__ float act_small(float v, int act) {
  switch (act) {
    case kActRelu: return fmaxf(v, 0.f);
    case kActSilu: return v * __fdividef(1.f, 1.f + __expf(-v));
    case kActGelu: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    default: return v;
  }
}

template <int NT, int SL, bool SWIGLU, bool BF16>
__global__ void __launch_bounds__(kWarps * 32) sparse_gemm_small_m_kernel(const SmallParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int kRows = 16 * SL;
  constexpr int kStages = kStagesFor(SL);
  constexpr int kWarpBytes = kWarpSmemFor(SL);
  float* red = reinterpret_cast<float*>(smem + kWarps * kWarpBytes);   // [kWarps][kRows][8*NT]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t wbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem + warp * kWarpBytes));

  // this warp's share of the 128-wide K tiles
  const int kt_lo = (p.k_tiles128 * warp) / kWarps;
  const int kt_hi = (p.k_tiles128 * (warp + 1)) / kWarps;
  const int n_kt = kt_hi - kt_lo;
  const int kc_total = p.K / 2;   // compressed elements per row

  // X fragment cache of this warp's K slice: xs[(k-step * NT + n) * 32 + lane] = (b0, b1, b2, b3)
  uint4* xs = nullptr;
  if (p.xs_ksteps > 0) {
    uint8_t* xs_base = smem + kWarps * kWarpBytes + 2 * kWarps * kRows * 8 * NT * 4;
    xs = reinterpret_cast<uint4*>(xs_base) + static_cast<size_t>(warp) * p.xs_ksteps * NT * 32;
    for (int ks = 0; ks < n_kt * 4; ++ks) {
      const int k0 = (kt_lo * 4 + ks) * 32;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int tok = n * 8 + g;
        uint4 bv = make_uint4(0u, 0u, 0u, 0u);
        if (tok < p.m_tok && k0 < p.K) {
          const uint32_t* xp = reinterpret_cast<const uint32_t*>(p.x + static_cast<size_t>(tok) * p.ldx + k0 + 2 * t);
          bv = make_uint4(__ldg(xp), __ldg(xp + 4), __ldg(xp + 8), __ldg(xp + 12));
        }
        xs[(ks * NT + n) * 32 + lane] = bv;
      }
    }
    __syncwarp();
  }

  // The cp.async ring runs continuously over this warp's (slab, k-tile) items, so the loads of the
  // next slab are in flight while the current one is reduced.
  const int my_slabs = (p.num_slabs - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);
  const int total_items = my_slabs * n_kt;
  // issue cursor (slab, k-tile, ring slot) advances incrementally: no divisions in the loop
  int issued = 0, iss_slab = blockIdx.x, iss_kt = 0, iss_slot = 0, con_slot = 0;
  auto issue_next = [&]() {
    if (issued < total_items) {
      const int kt = kt_lo + iss_kt;
      const int kc0 = kt * 64;   // first compressed element of the chunk
      const int r0 = iss_slab * kRows;
      const uint32_t sdst = wbase + iss_slot * SL * kStageBytes;
#pragma unroll
      for (int j = 0; j < 4 * SL; ++j) {
        const int idx = j * 32 + lane;
        const int r = idx >> 3, c16 = idx & 7;
        const int row = r0 + r;
        const bool ok = row < p.n_out && kc0 + c16 * 8 < kc_total;
        const uint16_t* src = p.values + static_cast<size_t>(ok ? row : 0) * kc_total + (ok ? kc0 + c16 * 8 : 0);
        cp_async16(sdst + (r >> 4) * kValBytes + (r & 15) * kRowPitch + c16 * 16, src, ok);
      }
      if (lane < 16 * SL) {   // metadata: lanes [16*m2, 16*m2+16) of the 128-lane tile, 16 B each
        const int sl = lane >> 4, ln = lane & 15;
        const int r16 = r0 + 16 * sl;
        const uint32_t* mp = p.meta + ((static_cast<size_t>(r16 >> 7) * p.k_tiles128 + kt) * 128 +
                                       (((r16 & 127) >> 4) * 16 + ln)) * 4;
        cp_async16(sdst + SL * kValBytes + sl * 256 + ln * 16, mp, true);
      }
      if (++iss_kt == n_kt) { iss_kt = 0; iss_slab += gridDim.x; }
    }
    cp_async_commit();
    ++issued;
    if (++iss_slot == kStages) iss_slot = 0;
  };
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) issue_next();

  // L1 path for X (used when the fragment cache does not fit): fragments of one k-tile
  uint32_t bnext[4][NT][4];
  auto load_b = [&](int kt, uint32_t (&dst)[4][NT][4]) {
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      const int k0 = kt * 128 + kb * 32;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int tok = n * 8 + g;
        const bool ok = tok < p.m_tok && k0 < p.K;
        const uint32_t* xp = reinterpret_cast<const uint32_t*>(p.x + static_cast<size_t>(ok ? tok : 0) * p.ldx + (ok ? k0 : 0) + 2 * t);
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[kb][n][q] = ok ? __ldg(xp + 4 * q) : 0u;
      }
    }
  };
  if (xs == nullptr && n_kt > 0) load_b(kt_lo, bnext);

  int parity = 0;
  for (int slab = blockIdx.x; slab < p.num_slabs; slab += gridDim.x, parity ^= 1) {
    const int row0 = slab * kRows;
    float acc[SL][NT][4];
#pragma unroll
    for (int sl = 0; sl < SL; ++sl)
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[sl][n][i] = 0.f;

    for (int i = 0; i < n_kt; ++i) {
      issue_next();
      cp_async_wait<kStages - 1>();
      __syncwarp();
      // metadata: lanes with t < 2 hold the four words (one per 32-wide K block) of rows g, g+8
      uint32_t e4[SL][4];
      const uint32_t sA = wbase + con_slot * SL * kStageBytes;
      const uint8_t* sA_gen = smem + warp * kWarpBytes + con_slot * SL * kStageBytes;
      if (++con_slot == kStages) con_slot = 0;
#pragma unroll
      for (int sl = 0; sl < SL; ++sl) {
        // lane (g, t < 2) takes tile lane g + 8t: rows g and g+8, K half t
        const uint4 mw = *reinterpret_cast<const uint4*>(sA_gen + SL * kValBytes + sl * 256 + (g + 8 * (t & 1)) * 16);
        e4[sl][0] = mw.x; e4[sl][1] = mw.y; e4[sl][2] = mw.z; e4[sl][3] = mw.w;
      }
      // B fragments of this k-tile: from the shared-memory cache, or from the registers that were
      // loaded through L1 one k-tile ahead
      uint32_t bcur[4][NT][4];
#pragma unroll
      for (int kb = 0; kb < 4; ++kb)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          if (xs != nullptr) {
            const uint4 bv = xs[((i * 4 + kb) * NT + n) * 32 + lane];
            bcur[kb][n][0] = bv.x; bcur[kb][n][1] = bv.y; bcur[kb][n][2] = bv.z; bcur[kb][n][3] = bv.w;
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) bcur[kb][n][q] = bnext[kb][n][q];
          }
        }
      if (xs == nullptr) load_b(kt_lo + (i + 1 < n_kt ? i + 1 : 0), bnext);   // next k-tile (wraps to the next slab's first)
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {
        uint32_t a[SL][4];
        // matrices: (rows 0-7, c 0-7), (rows 8-15, c 0-7), (rows 0-7, c 8-15), (rows 8-15, c 8-15)
        const int mr = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int mc = (lane >> 4) * 8;
#pragma unroll
        for (int sl = 0; sl < SL; ++sl)
          ldmatrix_x4(sA + sl * kValBytes + mr * kRowPitch + (kb * 16 + mc) * 2, a[sl][0], a[sl][1], a[sl][2], a[sl][3]);
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int sl = 0; sl < SL; ++sl) mma_sp_16832<BF16>(acc[sl][n], a[sl], bcur[kb][n], e4[sl][kb]);
      }
      __syncwarp();
    }

    // cross-warp reduction: red[warp][row 0..kRows)[token 0..8NT)
    float* redp = red + parity * (kWarps * kRows * 8 * NT);   // double-buffered: one barrier per slab
    float* mine = redp + warp * kRows * 8 * NT;
#pragma unroll
    for (int sl = 0; sl < SL; ++sl)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        float* base = mine + (16 * sl) * 8 * NT + n * 8 + 2 * t;
        base[g * 8 * NT] = acc[sl][n][0];
        base[g * 8 * NT + 1] = acc[sl][n][1];
        base[(g + 8) * 8 * NT] = acc[sl][n][2];
        base[(g + 8) * 8 * NT + 1] = acc[sl][n][3];
      }
    __syncthreads();
    constexpr int kOutRows = SWIGLU ? 16 : kRows;
    for (int i = threadIdx.x; i < kOutRows * 8 * NT; i += kWarps * 32) {
      // consecutive threads -> consecutive rows, so stores of one token are contiguous
      const int r = i % kOutRows, tok = i / kOutRows;
      float s = 0.f, s2 = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        s += redp[w * kRows * 8 * NT + r * 8 * NT + tok];
        if (SWIGLU) s2 += redp[w * kRows * 8 * NT + (r + 16) * 8 * NT + tok];
      }
      if (tok >= p.m_tok) continue;
      if (SWIGLU) {
        const int f = slab * 16 + r;                      // hidden feature
        if (f < p.n_out / 2) {
          const float h = (s * __fdividef(1.f, 1.f + __expf(-s))) * s2;
          p.y[static_cast<size_t>(tok) * p.ldy + f] =
              BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(h)) : __half_as_ushort(__float2half_rn(h));
        }
      } else {
        const int row = row0 + r;
        if (row < p.n_out) {
          if (p.bias) s += BF16 ? __uint_as_float(static_cast<uint32_t>(p.bias[row]) << 16)
                                : __half2float(__ushort_as_half(p.bias[row]));
          s = act_small(s, p.act);
          p.y[static_cast<size_t>(tok) * p.ldy + row] =
              BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(s)) : __half_as_ushort(__float2half_rn(s));
        }
      }
    }
  }
  cp_async_wait<0>();
}

template <int NT, int SL, bool SWIGLU, bool BF16>
int launch_nt(SmallParams p, int num_sms, cudaStream_t stream) {
  int smem = kWarps * kWarpSmemFor(SL) + 2 * kWarps * 16 * SL * 8 * NT * 4;
  {  // X fragment cache if it leaves room (k-steps per warp x NT x 512 B x 8 warps)
    const int ksteps = ((p.k_tiles128 + kWarps - 1) / kWarps) * 4;
    const int xs_bytes = kWarps * ksteps * NT * 512;
    p.xs_ksteps = (smem + xs_bytes <= 200 * 1024) ? ksteps : 0;
    if (p.xs_ksteps) smem += xs_bytes;
  }
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(sparse_gemm_small_m_kernel<NT, SL, SWIGLU, BF16>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return kErrCuda;
    attr_set[dev] = true;
  }
  // resident CTAs per SM: the count (1 or 2) that needs the fewest bandwidth-rounds
  const long units = p.num_slabs;
  const long r1 = (units + num_sms - 1) / num_sms, r2 = (units + 2L * num_sms - 1) / (2L * num_sms);
  const bool two = smem <= 110 * 1024 && 2 * r2 <= r1;
  long ctas = static_cast<long>(num_sms) * (two ? 2 : 1);
  if (ctas > units) ctas = units;
  sparse_gemm_small_m_kernel<NT, SL, SWIGLU, BF16>
      <<<static_cast<int>(ctas), kWarps * 32, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

template <int SL, bool SWIGLU>
int dispatch_nt(const SmallParams& p, int nt, bool bf, int num_sms, cudaStream_t stream) {
  switch (nt) {
    case 1: return bf ? launch_nt<1, SL, SWIGLU, true>(p, num_sms, stream) : launch_nt<1, SL, SWIGLU, false>(p, num_sms, stream);
    case 2: return bf ? launch_nt<2, SL, SWIGLU, true>(p, num_sms, stream) : launch_nt<2, SL, SWIGLU, false>(p, num_sms, stream);
    case 3: return bf ? launch_nt<3, SL, SWIGLU, true>(p, num_sms, stream) : launch_nt<3, SL, SWIGLU, false>(p, num_sms, stream);
    default: return bf ? launch_nt<4, SL, SWIGLU, true>(p, num_sms, stream) : launch_nt<4, SL, SWIGLU, false>(p, num_sms, stream);
  }
}

}  // namespace

int launch_sparse_gemm_small_m(const SparseGemmArgs& a, cudaStream_t stream) {
  if (a.m_tok <= 0 || a.m_tok > 8 * kMaxNT || a.K % 64 != 0 || a.n_out <= 0) return kErrInvalid;
  if (a.ldx % 2 != 0 || (reinterpret_cast<uintptr_t>(a.x) & 3) || (reinterpret_cast<uintptr_t>(a.values) & 15) ||
      (reinterpret_cast<uintptr_t>(a.meta) & 15) || (a.K / 2) % 8 != 0)
    return kErrInvalid;
  if (a.epi == kEpiSwiGLU && a.n_out % 32 != 0) return kErrInvalid;
  SmallParams p;
  p.x = static_cast<const uint16_t*>(a.x);
  p.values = static_cast<const uint16_t*>(a.values);
  p.meta = static_cast<const uint32_t*>(a.meta);
  p.bias = static_cast<const uint16_t*>(a.bias);
  p.y = static_cast<uint16_t*>(a.y);
  p.m_tok = a.m_tok;
  p.n_out = a.n_out;
  p.K = a.K;
  p.ldx = a.ldx;
  p.ldy = a.ldy;
  p.k_tiles128 = (a.K + 127) / 128;
  p.fmt = a.fmt;
  p.act = a.act;
  p.xs_ksteps = 0;
  const int nt = (a.m_tok + 7) / 8;
  const bool bf = a.fmt == kBF16;
  if (a.epi == kEpiSwiGLU) {
    p.num_slabs = a.n_out / 32;
    return dispatch_nt<2, true>(p, nt, bf, a.num_sms, stream);
  }
  p.num_slabs = (a.n_out + 15) / 16;
  return dispatch_nt<1, false>(p, nt, bf, a.num_sms, stream);
}

}  // namespace sfb200
