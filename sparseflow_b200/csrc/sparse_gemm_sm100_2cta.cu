// 2:4-sparse GEMM for sm_100a, CTA-pair variant for prefill-sized token counts.
//
// Same math and operand formats as sparse_gemm_sm100.cu, but two CTAs (a cluster of 2, on an SM
// pair) work on one tile of (256 * RS) weight rows x BN tokens with tcgen05.mma.sp.cta_group::2:
//   * each CTA holds RS sub-tiles of 128 weight rows (compressed values + metadata) and HALF of
//     the token tile; per k-block it issues RS MMAs (M = 256 across the pair, N = BN) that share
//     the token operand.  What this buys is bytes: the kernel is bound by what L2 can feed the
//     SMs, and a tile of R rows x T tokens moves R*K + 2*T*K bytes for 2*R*T*K flops, i.e.
//     2RT/(R+2T) flop/B: 96-102 for the single-CTA 128x192/256 tiles, 171 for 256x256 (RS = 1),
//     229 for 512x208 (RS = 2).  Shared-memory reads per MMA drop the same way (each SM reads half
//     of the token tile);
//   * the even CTA of the pair issues every MMA; completion is signalled to both CTAs;
//   * accumulators (RS x BN fp32 columns, 128 lanes per CTA) live in tensor memory, which has 512
//     columns of which the metadata ring needs 16-32.  With RS = 1 and BN <= 240 two accumulators
//     fit (2 x 240 + 16 = 496): the MMA stream of tile i+1 fills one while the epilogue drains the
//     other, so the epilogue is off the critical path.  BN = 256 and the RS = 2 tiles have a single
//     accumulator set: the MMA stream waits for their drain, which is therefore spread over sixteen
//     warps instead of eight.
//
// Warps: warp 0 = TMA producer, warp 1 = MMA issuer / tensor-memory owner, warps 2 and up = epilogue
// (8 or 16).  The drain is one rolled loop over 16-column chunks for every tile.
// All loads are plain per-CTA TMA copies; nothing here reads another GPU's memory.
#include <cmath>
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
// Arrive on a barrier of the pair's even CTA.  Default semantics (release at CTA scope) on purpose:
// a cluster-scope release would hold the arrive back until this thread's global stores of the
// previous tile have reached L2, and the arrive only has to order tensor-memory reads, which
// tcgen05.wait::ld + tcgen05.fence::before_thread_sync already do.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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
// L2 eviction policies: outputs are written once and never read by this kernel (evict first, so
// they do not push operand tiles out of L2); the token operand is re-read by every row block
// (evict last).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst, const CUtensorMap* m, int x, int y,
                                                      uint32_t leader_bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(leader_bar), "l"(policy)
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
  int num_m_blks, num_n_blks;   // (256*RS)-row / BN-token tiles
  int k_tiles128;
  int fmt, act;
  int tok_per_owner;   // > 0: token block o (tok_per_owner tokens) is stored to peer_y[o] instead of y (reduce-scatter
                       // fused into the epilogue: peer_y[o] = rank o's receive slot for this rank's partial sums)
  void* peer_y[8];
  int band;            // tiles of the RESIDENT operand per L2 band (see tile_coords)
  int order;           // 0: activations resident (bands of token tiles); 1: weights resident (bands of row tiles)
  int n_rot;           // token tiles are visited starting from this one (wrapping around): with the reduce-scatter in the
                       // epilogue every rank starts at another owner's block, so no owner receives from all ranks at once
  int out_f32;         // store epilogue: 1 = y is float [m_tok, ldy], results stored unrounded; 2 = y is fp16 whatever
                       // the operand type, results clamped to the finite fp16 range (partial sums on their way to a sum)
};

// Tile order.  The SM pairs run in lockstep along K, so data shared by the tiles of one pass over the SMs
// ("wave") is fetched from HBM once; what decides the L2 hit rate is whether the operand that the NEXT
// wave needs again is still there.  One operand is therefore kept resident (loaded with an evict-last
// hint) and the other is streamed: the resident operand is cut into bands of about 56 MB, and inside a band
// the tiles of the streamed operand are the slow index, so that every wave touches the whole band of the
// resident operand and only a few tiles of the streamed one.
//   order 0: activations resident (bands of token tiles, row tile slow inside a band): gate|up-like shapes,
//            where the activations are the smaller operand;
//   order 1: weights resident (bands of row tiles, token tile slow inside a band): down-projection-like
//            shapes (long K, few rows), where hidden[M, I] is larger than the compressed weight.  (Measured on
//            4096 x 11008 at 4096 tokens with order 0: 72 % L2 hit rate, 325 MB read from HBM for 140 MB of
//            operands; the gate|up shape, whose activations fit, runs at 94 %.)
__device__ __forceinline__ void tile_coords(int tile, const PairParams& p, int& m_blk, int& n_blk) {
  if (p.order == 0) {
    const int per_band = p.num_m_blks * p.band;
    const int b = tile / per_band;
    const int r = tile - b * per_band;
    const int left = p.num_n_blks - b * p.band;
    const int width = left < p.band ? left : p.band;
    m_blk = r / width;
    n_blk = b * p.band + (r - m_blk * width);
  } else {
    const int per_band = p.num_n_blks * p.band;
    const int b = tile / per_band;
    const int r = tile - b * per_band;
    const int left = p.num_m_blks - b * p.band;
    const int height = left < p.band ? left : p.band;
    n_blk = r / height;
    m_blk = b * p.band + (r - n_blk * height);
  }
  n_blk += p.n_rot;
  if (n_blk >= p.num_n_blks) n_blk -= p.num_n_blks;
}

int g_force_order = -1;  // tuning hook: -1 automatic, 0 / 1 force the tile order
int g_l2_band_mb = 56;   // budget of the resident operand's band (tuning hook: set_l2_band_mb)

// Tiles of the resident operand per band: `per_blk` bytes each, `count` of them in all.
inline int pick_band(long per_blk, int count) {
  long band = (static_cast<long>(g_l2_band_mb) << 20) / (per_blk > 0 ? per_blk : 1);
  if (band < 1) band = 1;
  if (band >= count) return count;
  // equal bands: avoid a narrow last band
  const long nb = (count + band - 1) / band;
  band = (count + nb - 1) / nb;
  return static_cast<int>(band);
}

// Which operand stays resident, and the band size, for a rows x K weight against m_tok tokens.
inline void pick_order(int n_out, int m_tok, int K, int rows_tile, int bn, int num_m_blks, int num_n_blks,
                       PairParams& p) {
  const double w_bytes = static_cast<double>(n_out) * K * 1.125, x_bytes = static_cast<double>(m_tok) * K * 2.0;
  if (w_bytes < x_bytes) {
    p.order = 1;
    p.band = pick_band(static_cast<long>(rows_tile * 1.125 * K), num_m_blks);
  } else {
    p.order = 0;
    p.band = pick_band(static_cast<long>(bn) * K * 2, num_n_blks);
  }
}

template <int BN_, int BK_, int STAGES_, int RS_, int EPI_>
struct PairCfg {
  static constexpr int BN = BN_;         // tokens per tile (pair-wide)
  static constexpr int BK = BK_;
  static constexpr int STAGES = STAGES_;
  static constexpr int RS = RS_;         // 128-row sub-tiles per CTA
  static constexpr int EPI = EPI_;
  static constexpr int ROWS_CTA = 128 * RS;
  static constexpr int ROWS_TILE = 2 * ROWS_CTA;
  static constexpr int HALF_N = BN / 2;  // tokens loaded by each CTA
  static constexpr int A_SUB_BYTES = 128 * (BK / 2) * 2;
  static constexpr int A_BYTES = RS * A_SUB_BYTES;
  static constexpr int B_SUBS = BK / 64;
  static constexpr int B_SUB_BYTES = HALF_N * 128;
  static constexpr int B_BYTES = B_SUBS * B_SUB_BYTES;
  static constexpr int E_SUB_BYTES = 2048;
  static constexpr int E_BYTES = RS * E_SUB_BYTES;
  static constexpr int MMAS_PER_STAGE = BK / 32;
  // Metadata tiles cover K = 128: with BK = 64 one tile serves two stages, so the metadata ring
  // (shared memory and tensor-memory columns) has STAGES/2 + 1 slots.  A slot is reused
  // STAGES + 2 stages after it was written, i.e. after the stage barrier that guards it.
  static constexpr int E_STAGES = (BK == 128) ? STAGES : STAGES / 2 + 1;
  static constexpr int E_COLS_STAGE = 4 * RS;
  // accumulator sets: two when they fit beside the metadata ring (RS = 1, BN <= 240)
  static constexpr int ACC_COLS = RS * BN;
  static constexpr int ACC_BUFS = (RS == 1 && 2 * ACC_COLS + E_COLS_STAGE * E_STAGES <= 512) ? 2 : 1;
  static constexpr int E_COL0 = ACC_BUFS * ACC_COLS;   // metadata columns start after the accumulators
  static constexpr int TMEM_USED = ACC_BUFS * ACC_COLS + E_COLS_STAGE * E_STAGES;
  static constexpr int TMEM_COLS = TMEM_USED <= 128 ? 128 : TMEM_USED <= 256 ? 256 : 512;
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + STAGES * A_BYTES;
  static constexpr int OFF_E = OFF_B + STAGES * B_BYTES;
  // per-warp output staging for the register-drain epilogue: 2 buffers of 16 tokens x
  // 32 rows (or 16 features for SiLU.mul) of 16-bit values
  static constexpr int D_ROW_BYTES = (EPI == kEpiSwiGLU) ? 32 : 64;
  static constexpr int D_BUF_BYTES = 16 * D_ROW_BYTES;
  static constexpr int OFF_D = OFF_E + E_STAGES * E_BYTES;
  // Epilogue warps: 4 lane quadrants x 2 where the tile has two accumulator sets (its drain hides behind the next tile's
  // K loop), x 4 where it has one (256 x 256 and the 512-row tiles: the MMA stream waits for the drain, and a 16-column
  // chunk is a chain of a few hundred dependent instructions, so what shortens the drain is more warps per scheduler).
  // The warps of a quadrant share the accumulator's 16-column chunks: RS = 2 -> one row set each, then halves.
  static constexpr int EPI_WARPS = (ACC_BUFS == 1) ? 16 : 8;
  static constexpr int D_BUFS = (EPI_WARPS == 16) ? 1 : 2;
  static constexpr int D_BYTES = EPI_WARPS * D_BUFS * D_BUF_BYTES;
  static constexpr int OFF_BAR = OFF_D + D_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int CHUNKS = BN / 16;
  static constexpr int PARTS = EPI_WARPS / 4 / RS;                  // warps that share one accumulator's chunks
  static constexpr int CHUNKS_PER_PART = (CHUNKS + PARTS - 1) / PARTS;
  static_assert((PARTS - 1) * CHUNKS_PER_PART < CHUNKS, "every epilogue warp has at least one chunk");
  static_assert(RS == 1 || RS == 2, "RS");
  static_assert(BK == 128 || STAGES % 2 == 0, "BK = 64 needs an even stage count");
  static_assert(BN % 16 == 0 && BN <= 256 && BN >= 128, "BN");
  static_assert(HALF_N % 8 == 0, "token half must be whole swizzle atoms");
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
__device__ __forceinline__ float bias_at(const void* bias, int o, int fmt) {
  const uint16_t b = static_cast<const uint16_t*>(bias)[o];
  if (fmt == 1) return __uint_as_float(static_cast<uint32_t>(b) << 16);
  return __half2float(__ushort_as_half(b));
}
// 16 lanes x 16 columns: thread l gets, for repetition n (8 columns each), r[4n], r[4n+1] =
// (lane l/4, columns 8n + 2(l%4), +1) and r[4n+2], r[4n+3] = (lane l/4 + 8, same columns): the
// accumulator-fragment layout of warp-level MMA, which stmatrix can transpose.  Two repetitions: 8 registers.
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
// 32 lanes x 16 columns of fp32: thread i = lane base + i, one register per column
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2,
                                                  uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(addr),
               "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}
__device__ __forceinline__ uint32_t pack16(float a, float b, int fmt) {
  if (fmt == 1) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float silu_mul(uint32_t g, uint32_t u) {
  const float gf = __uint_as_float(g);
  return (gf * __fdividef(1.f, 1.f + __expf(-gf))) * __uint_as_float(u);
}

template <class C>
__device__ __forceinline__ void pair_kernel_body(const CUtensorMap& tmA, const CUtensorMap& tmB,
                                                 const CUtensorMap& tmE, const PairParams& p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  const uint32_t bar_full = smem_u32(bars);                 // used in the even CTA only
  const uint32_t bar_empty = bar_full + 8 * C::STAGES;      // both CTAs
  const uint32_t bar_accf = bar_empty + 8 * C::STAGES;      // both CTAs, one per accumulator set
  const uint32_t bar_acce = bar_accf + 16;                  // even CTA only, one per accumulator set
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + 8 * (2 * C::STAGES + 4));
  volatile int* err = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_tiles = p.num_m_blks * p.num_n_blks;
  // With BK = 64 the k loop always runs an even number of stages (a trailing stage beyond K loads
  // zero-filled operands), so metadata loads fall on every second stage without exception.
  const int k_iters = (C::BK == 128) ? (p.K + 127) / 128 : 2 * ((p.K + 127) / 128);

  if (threadIdx.x == 0) {
    *err = 0;
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_accf + 8 * b, 1);
      mbar_init(bar_acce + 8 * b, 2 * C::EPI_WARPS);
    }
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
      const uint64_t pol_keep = l2_policy_evict_last();
      const bool keep_x = p.order == 0;      // the resident operand is loaded evict-last, the streamed one plainly
      int s = 0, es = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        int m_blk, n_blk;
        tile_coords(tile, p, m_blk, n_blk);
        const int row0 = m_blk * C::ROWS_TILE + static_cast<int>(rank) * C::ROWS_CTA;
        const int tok0 = n_blk * C::BN + static_cast<int>(rank) * C::HALF_N;
        const int e_rt0 = row0 >> 7;   // first 128-row metadata tile of this CTA
        for (int kt = 0; kt < k_iters; ++kt) {
          ok = mbar_wait(bar_empty + 8 * s, ph ^ 1, err, p.status, 1);
          if (!ok) break;
          const bool load_e = (C::BK == 128) || ((kt & 1) == 0);
          const uint32_t full = leader_full0 + 8 * s;
          if (leader)   // bytes of BOTH CTAs land on this barrier
            mbar_arrive_expect_tx(bar_full + 8 * s,
                                  2 * (C::A_BYTES + C::B_BYTES + (load_e ? C::E_BYTES : 0)));
          // one copy per 128-row sub-tile
#pragma unroll
          for (int rs = 0; rs < C::RS; ++rs) {
            const uint32_t dst = sbase + C::OFF_A + s * C::A_BYTES + rs * C::A_SUB_BYTES;
            if (keep_x) tma_load_2d_pair(dst, &tmA, kt * (C::BK / 2), row0 + 128 * rs, full);
            else tma_load_2d_pair_hint(dst, &tmA, kt * (C::BK / 2), row0 + 128 * rs, full, pol_keep);
          }
#pragma unroll
          for (int j = 0; j < C::B_SUBS; ++j) {
            const uint32_t dst = sbase + C::OFF_B + s * C::B_BYTES + j * C::B_SUB_BYTES;
            if (keep_x) tma_load_2d_pair_hint(dst, &tmB, kt * C::BK + j * 64, tok0, full, pol_keep);
            else tma_load_2d_pair(dst, &tmB, kt * C::BK + j * 64, tok0, full);
          }
          if (load_e) {
            const int kt128 = (C::BK == 128) ? kt : (kt >> 1);
#pragma unroll
            for (int rs = 0; rs < C::RS; ++rs)
              tma_load_1d_pair(sbase + C::OFF_E + es * C::E_BYTES + rs * C::E_SUB_BYTES, &tmE,
                               ((e_rt0 + rs) * p.k_tiles128 + kt128) * 256, full);
            if (++es == C::E_STAGES) es = 0;
          }
          if (++s == C::STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (leader && elect_one()) {
      const uint32_t idesc = make_idesc_f16(256, C::BN, p.fmt, true);
      int s = 0, es = 0;
      uint32_t ph = 0;
      uint32_t e_cols = 0;
      bool ok = true;
      uint32_t it = 0;    // tiles done by this pair: accumulator set = it % ACC_BUFS, its use count = it / ACC_BUFS
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++it) {
        const uint32_t as = (C::ACC_BUFS == 2) ? (it & 1u) : 0u;
        const uint32_t use = (C::ACC_BUFS == 2) ? (it >> 1) : it;
        const uint32_t d_base = tmem_base + as * C::ACC_COLS;
        ok = mbar_wait(bar_acce + 8 * as, (use & 1u) ^ 1u, err, p.status, 3);
        if (!ok) break;
        tc_fence_after();
        for (int kt = 0; kt < k_iters; ++kt) {
          ok = mbar_wait(bar_full + 8 * s, ph, err, p.status, 2);
          if (!ok) break;
          tc_fence_after();
          const bool new_e = (C::BK == 128) || ((kt & 1) == 0);
          if (new_e) {
            e_cols = C::E_COL0 + C::E_COLS_STAGE * es;
#pragma unroll
            for (int rs = 0; rs < C::RS; ++rs)
              tc_cp_128x128b_pair(tmem_base + e_cols + 4 * rs,
                                  make_smem_desc(sbase + C::OFF_E + es * C::E_BYTES + rs * C::E_SUB_BYTES, 0,
                                                 128, kSwNone));
            if (++es == C::E_STAGES) es = 0;
          }
          const uint32_t a_addr = sbase + C::OFF_A + s * C::A_BYTES;
          const uint32_t b_addr = sbase + C::OFF_B + s * C::B_BYTES;
#pragma unroll
          for (int kb = 0; kb < C::MMAS_PER_STAGE; ++kb) {
            const uint64_t bdesc = make_smem_desc(
                b_addr + (kb >> 1) * C::B_SUB_BYTES + (kb & 1) * 64, 16, 1024, kSw128);
            const int ecol = (C::BK == 128) ? kb : ((kt & 1) * 2 + kb);
#pragma unroll
            for (int rs = 0; rs < C::RS; ++rs) {
              const uint32_t a_sub = a_addr + rs * C::A_SUB_BYTES + kb * 32;
              const uint64_t adesc = (C::BK == 64) ? make_smem_desc(a_sub, 16, 512, kSw64)
                                                   : make_smem_desc(a_sub, 16, 1024, kSw128);
              tc_mma_sp_f16_pair(d_base + rs * C::BN, adesc, bdesc,
                                 tmem_base + e_cols + 4 * rs + (ecol & ~1), idesc | (ecol & 1),
                                 (kt > 0 || kb > 0) ? 1u : 0u);
            }
          }
          tc_commit_pair(bar_empty + 8 * s);
          if (++s == C::STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        tc_commit_pair(bar_accf + 8 * as);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2 and up, both CTAs)
    const int q = warp & 3;                 // lane quadrant
    const int w2 = (warp - 2) >> 2;         // index of this warp among the warps of its quadrant
    const int acc = (C::RS == 1) ? 0 : (w2 & 1);                    // row set
    const int part = (C::RS == 1) ? w2 : (w2 >> 1);
    // chunks [c_begin, c_end) of the accumulator are this warp's to store
    const int c_begin = part * C::CHUNKS_PER_PART;
    const int c_end = c_begin + C::CHUNKS_PER_PART < C::CHUNKS ? c_begin + C::CHUNKS_PER_PART : C::CHUNKS;
    const uint32_t leader_acce0 = mapa_u32(bar_acce, 0);
    const uint64_t pol_stream = l2_policy_evict_first();
    bool ok = true;
    uint32_t it = 0;
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++it) {
      int m_blk, n_blk;
      tile_coords(tile, p, m_blk, n_blk);
      const uint32_t as = (C::ACC_BUFS == 2) ? (it & 1u) : 0u;
      const uint32_t use = (C::ACC_BUFS == 2) ? (it >> 1) : it;
      const uint32_t leader_acce = leader_acce0 + 8 * as;
      {
        bool w = mbar_wait(bar_accf + 8 * as, use & 1u, err, p.status, 4);
        ok = __all_sync(0xffffffffu, w);
      }
      if (!ok) break;
      tc_fence_after();
      const int row_w = m_blk * C::ROWS_TILE + static_cast<int>(rank) * C::ROWS_CTA + acc * 128 + q * 32;
      const int tok_w = n_blk * C::BN;
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * C::ACC_COLS + acc * C::BN;
      // The drain is a ROLLED loop over 16-column chunks (load, wait, convert, store; ~150 instructions).  The epilogue's
      // code is executed once per tile by warps that are out of step with one another, and a drain written out in full
      // (128 accumulator registers converted and stored one by one, thousands of instructions) ran out of the
      // instruction cache: measured 17-35 stall cycles per issued instruction for every warp of the SM, the TMA producer
      // and the MMA issuer included (512 x 240 tile on 4096 x 11008 at 2048 tokens: tensor pipe active 28 %, 197 us;
      // rolled 75 us).  The accumulator is handed back as soon as its last chunk is in registers.
      const int out_cols = (C::EPI == kEpiSwiGLU) ? p.n_out / 2 : p.n_out;
      const int g = lane >> 2;
      const uint32_t stage0 = sbase + C::OFF_D + (warp - 2) * C::D_BUFS * C::D_BUF_BYTES;
      // stmatrix row address of this lane: matrix = lane / 8, row in matrix = lane % 8
      const int mt = lane >> 3, rr = lane & 7;
      const uint32_t st_off = static_cast<uint32_t>((rr + 8 * (mt >> 1)) * C::D_ROW_BYTES + 16 * (mt & 1));
      const int out_x = (C::EPI == kEpiSwiGLU) ? row_w / 2 : row_w;   // first output column of this warp

      // destination of the 16-token chunk that starts at token t0: the output tensor, or (row-parallel GEMM with the
      // reduce-scatter fused in) the receive slot of the rank that owns these tokens -- stores over NVLink
      auto chunk_dst = [&](int t0, int& tl) -> void* {
        tl = t0;
        if (C::EPI == kEpiStore && p.tok_per_owner > 0) {
          const int owner = t0 / p.tok_per_owner;
          tl = t0 - owner * p.tok_per_owner;
          return p.peer_y[owner < 8 ? owner : 7];
        }
        return p.y;
      };
      // 16-bit output of one chunk whose fragment registers are a[0..8) (lanes 0-15 of the quadrant) and b[0..8)
      // (lanes 16-31): transpose through the staging tile, then plain 16-byte stores.  (A TMA store per chunk queues
      // behind the producer's loads in the copy engine and its completion, which the staging buffer's reuse has to
      // wait for, takes longer than the chunk itself.)
      auto store_chunk16 = [&](const uint32_t* a, const uint32_t* b, int c, int t0, float b0, float b1, float b2, float b3) {
        const uint32_t stage = stage0 + (c & (C::D_BUFS - 1)) * C::D_BUF_BYTES;
        __syncwarp();                                 // every lane has read this buffer's previous contents
        if (C::EPI == kEpiSwiGLU) {
          // half 0 = 16 gate rows, half 1 = the 16 matching up rows: pairing is in-thread
          // (the output type is tested once per chunk, not once per value: the drain is a chain of dependent
          // instructions and every branch inside it costs latency that nothing hides)
          if (p.fmt == 1)
            stmatrix_x4_trans(stage + st_off, pack16(silu_mul(a[0], b[0]), silu_mul(a[1], b[1]), 1),
                              pack16(silu_mul(a[2], b[2]), silu_mul(a[3], b[3]), 1),
                              pack16(silu_mul(a[4], b[4]), silu_mul(a[5], b[5]), 1),
                              pack16(silu_mul(a[6], b[6]), silu_mul(a[7], b[7]), 1));
          else
            stmatrix_x4_trans(stage + st_off, pack16(silu_mul(a[0], b[0]), silu_mul(a[1], b[1]), 0),
                              pack16(silu_mul(a[2], b[2]), silu_mul(a[3], b[3]), 0),
                              pack16(silu_mul(a[4], b[4]), silu_mul(a[5], b[5]), 0),
                              pack16(silu_mul(a[6], b[6]), silu_mul(a[7], b[7]), 0));
        } else {
          const bool half_out = p.out_f32 == 2;
          // which conversion runs is tested once per chunk, not once per value: the drain is a chain of dependent
          // instructions and every branch inside it costs latency that nothing hides
          auto emit = [&](auto f, const int of) {
            stmatrix_x4_trans(stage + st_off, pack16(f(a[0], b0), f(a[1], b0), of), pack16(f(a[2], b1), f(a[3], b1), of),
                              pack16(f(a[4], b0), f(a[5], b0), of), pack16(f(a[6], b1), f(a[7], b1), of));
            stmatrix_x4_trans(stage + st_off + 32, pack16(f(b[0], b2), f(b[1], b2), of),
                              pack16(f(b[2], b3), f(b[3], b3), of), pack16(f(b[4], b2), f(b[5], b2), of),
                              pack16(f(b[6], b3), f(b[7], b3), of));
          };
          if (p.act == kActNone && !half_out && p.fmt == 1) {          // bf16, no activation
            emit([](uint32_t v, float bias) { return __uint_as_float(v) + bias; }, 1);
          } else if (p.act == kActNone && half_out) {                   // partial sums on their way to a sum, as fp16
            emit([](uint32_t v, float bias) { return fminf(fmaxf(__uint_as_float(v) + bias, -65504.f), 65504.f); }, 0);
          } else {
            const int of = half_out ? 0 : p.fmt;
            emit([&](uint32_t v, float bias) {
              const float r = act_fn(__uint_as_float(v) + bias, p.act);
              return half_out ? fminf(fmaxf(r, -65504.f), 65504.f) : r;
            }, of);
          }
        }
        int tl;
        uint16_t* base = static_cast<uint16_t*>(chunk_dst(t0, tl));
        __syncwarp();
        // lane -> (token of the chunk, 16-byte unit of its row); the second round is 32 / UNITS_PER_TOK tokens further on
        constexpr int UNITS_PER_TOK = C::D_ROW_BYTES / 16;          // 4 (store) or 2 (SiLU.mul)
        constexpr int ROUNDS = UNITS_PER_TOK / 2, TOK_PER_ROUND = 32 / UNITS_PER_TOK;
        const int tk0 = lane / UNITS_PER_TOK, part = lane % UNITS_PER_TOK;
        const int col = out_x + part * 8;
        uint16_t* dst = base + static_cast<size_t>(tl + tk0) * p.ldy + col;
        const uint32_t src = stage + tk0 * C::D_ROW_BYTES + part * 16;
#pragma unroll
        for (int j = 0; j < ROUNDS; ++j) {
          if (t0 + tk0 + j * TOK_PER_ROUND < p.m_tok && col < out_cols) {
            uint4 v;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                         : "r"(src + j * TOK_PER_ROUND * C::D_ROW_BYTES));
            asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(
                             dst + static_cast<size_t>(j * TOK_PER_ROUND) * p.ldy),
                         "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol_stream)
                         : "memory");
          }
        }
      };
      // fp32 output of one chunk (partial sums that are added across ranks before they are rounded): the 32x32b load
      // gives every thread ONE row and 16 consecutive tokens, so a warp's store of one token is 32 consecutive floats
      // = 128 contiguous bytes: no transposition, full-size writes also when the destination is another GPU.
      auto store_chunk32 = [&](const uint32_t* r, int t0, float bias_v, bool row_ok) {
        int tl;
        float* dst = static_cast<float*>(chunk_dst(t0, tl)) + static_cast<size_t>(tl) * p.ldy + row_w + lane;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (row_ok && t0 + j < p.m_tok) dst[static_cast<size_t>(j) * p.ldy] = act_fn(__uint_as_float(r[j]) + bias_v, p.act);
      };
      auto release_acc = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(leader_acce);
      };

      if (C::EPI == kEpiStore && p.out_f32 == 1) {
        const bool row_ok = row_w + lane < p.n_out;
        const float bias_v = (p.bias != nullptr && row_ok) ? bias_at(p.bias, row_w + lane, p.fmt) : 0.f;
        uint32_t r[16];
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          tmem_ld_32x32b_x16(t_acc + 16 * c, r);
          tmem_ld_wait();
          const int t0 = tok_w + c * 16;
          if (t0 < p.m_tok) store_chunk32(r, t0, bias_v, row_ok);
        }
        release_acc();
      } else {
        float b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;   // bias of rows g, g+8, 16+g, 24+g
        if (C::EPI == kEpiStore && p.bias != nullptr) {
          if (row_w + g < p.n_out) b0 = bias_at(p.bias, row_w + g, p.fmt);
          if (row_w + g + 8 < p.n_out) b1 = bias_at(p.bias, row_w + g + 8, p.fmt);
          if (row_w + g + 16 < p.n_out) b2 = bias_at(p.bias, row_w + g + 16, p.fmt);
          if (row_w + g + 24 < p.n_out) b3 = bias_at(p.bias, row_w + g + 24, p.fmt);
        }
        // two register sets in turn: the loads of chunk c + 1 are in flight while chunk c is converted and stored
        uint32_t ra[8], rb[8], sa[8], sb[8];
        auto load_chunk = [&](int c, uint32_t (&lo)[8], uint32_t (&hi)[8]) {
          tmem_ld_16x256b_x2(t_acc + 16 * c, lo);                                          // lanes q*32 + 0..15
          tmem_ld_16x256b_x2(t_acc + 16 * c + (static_cast<uint32_t>(16) << 16), hi);      // lanes q*32 + 16..31
        };
        load_chunk(c_begin, ra, rb);
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 2) {
          tmem_ld_wait();
          if (c + 1 < c_end) load_chunk(c + 1, sa, sb);
          else release_acc();                                  // last chunk is in registers
          store_chunk16(ra, rb, c, tok_w + c * 16, b0, b1, b2, b3);
          if (c + 1 < c_end) {
            tmem_ld_wait();
            if (c + 2 < c_end) load_chunk(c + 2, ra, rb);
            else release_acc();
            store_chunk16(sa, sb, c + 1, tok_w + (c + 1) * 16, b0, b1, b2, b3);
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
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(C::THREADS, 1)
sparse_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmE, const PairParams p) {
  pair_kernel_body<C>(tmA, tmB, tmE, p);
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
  p.num_m_blks = (a.n_out + C::ROWS_TILE - 1) / C::ROWS_TILE;
  p.num_n_blks = (a.m_tok + C::BN - 1) / C::BN;
  p.k_tiles128 = (a.K + 127) / 128;
  p.fmt = a.fmt;
  p.act = a.act;
  p.tok_per_owner = 0;
  for (int o = 0; o < 8; ++o) p.peer_y[o] = nullptr;
  if (a.peer_y != nullptr) {      // row-parallel GEMM with the reduce-scatter fused into the epilogue
    if (C::EPI != kEpiStore || a.tp < 2 || a.tp > 8 || a.tok_per_owner <= 0 || a.tok_per_owner % 16 != 0 ||
        static_cast<long>(a.tok_per_owner) * a.tp < a.m_tok)
      return kErrInvalid;
    for (int o = 0; o < 8; ++o) {
      void* base = a.peer_y[o < a.tp ? o : 0];
      if (!base || (reinterpret_cast<uintptr_t>(base) & 15)) return kErrInvalid;
      p.peer_y[o] = base;
    }
    p.tok_per_owner = a.tok_per_owner;
  }
  p.out_f32 = a.out_f32;
  p.n_rot = 0;
  if (a.peer_y != nullptr && a.tp > 1 && a.tok_per_owner > 0) {
    const int first = ((a.rank + 1) % a.tp) * a.tok_per_owner / C::BN;   // the token tile where the next rank's block begins
    p.n_rot = first < p.num_n_blks ? first : 0;
  }
  pick_order(a.n_out, a.m_tok, a.K, C::ROWS_TILE, C::BN, p.num_m_blks, p.num_n_blks, p);
  if (g_force_order >= 0) {
    p.order = g_force_order;
    p.band = p.order ? pick_band(static_cast<long>(C::ROWS_TILE * 1.125 * a.K), p.num_m_blks)
                     : pick_band(static_cast<long>(C::BN) * a.K * 2, p.num_n_blks);
  }
  const int tiles = p.num_m_blks * p.num_n_blks;
  int pairs = a.num_sms / 2;
  if (pairs > tiles) pairs = tiles;
  if (pairs < 1) pairs = 1;
  sparse_gemm_pair_kernel<C><<<2 * pairs, C::THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, tmE, p);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

// Tile choice among the variants of dispatch_pair: estimated kernel time in microseconds from measurements on B200.
//   256-row x bn tile with two accumulator sets (12xx): a 128-wide K step costs 0.159 + 0.00102 * bn us (a constant
//     part for the weight tile plus a part per token column; the drain is hidden behind the next tile), 5 % more when
//     the activations are the streamed operand (tile order 1: few rows, long K -- the down projections), and 8 % more
//     per doubling of K above 4096, up to 12 % (measured per step, 240-token tile: 0.404 us on 22016 x 4096, 0.43 - 0.44
//     on 57344 x 8192 and 8192 x 8192, 0.45 - 0.47 on 4096 x 11008 / 14336, 0.48 on 8192 x 28672);
//   512-row tiles (52xx: 3 stages of K = 128, one accumulator set of 2 x bn columns, sixteen epilogue warps): the token
//     tile is written to shared memory once and read by two row sets, 0.247 + 0.00199 * bn us per K step whatever the
//     order, + 4 us of exposed drain per tile with the plain store epilogue, 1.5 us with SiLU.mul (half as much to
//     store): they win where K is long (4096 x 11008 at 4096 tokens 161 -> 142 us, 4096 x 14336 210 -> 188 us,
//     8192 x 28672 834 -> 735 us) and tie on the gate|up shapes of K = 4096;
//   256 x 256 with one accumulator set (1256, sixteen epilogue warps): the 12xx K step at bn = 256 + an exposed drain of
//     4 us (store) / 2 us (SiLU.mul) per tile; it wins where its 256-token tiles make one pass over the SM pairs and
//     the others need two (4096 x 11008 at 1024 tokens: 64 tiles, 46 us against 64 us for the next best);
//   launch, prologue, first fill and last drain: 8.5 us.
// What decides in practice is the number of passes over the SM pairs.
int pick_pair_variant_impl(int n_out, int m_tok, int K, int pairs, int swiglu, double* cost_us, bool hidden_drain = false) {
  const double k128 = (K + 127) / 128;
  const double dbl = k128 > 32.0 ? std::log2(k128 / 32.0) : 0.0;
  const double fk = 1.0 + 0.08 * (dbl < 1.5 ? dbl : 1.5);
  const bool x_streamed = static_cast<double>(n_out) * K * 1.125 < static_cast<double>(m_tok) * K * 2.0;   // as pick_order
  const double f12 = fk * (x_streamed ? 1.05 : 1.0);
  auto waves = [&](long tiles) { return static_cast<double>((tiles + pairs - 1) / pairs); };
  const long rows256 = (n_out + 255) / 256;
  double best_cost = 1e300;
  int best = 1240;
  const int cands[4] = {240, 224, 208, 192};
  for (int bn : cands) {
    const double c = 8.5 + waves(rows256 * ((m_tok + bn - 1) / bn)) * k128 * (0.159 + 0.00102 * bn) * f12;
    if (c < best_cost * 0.985) { best_cost = c; best = 1000 + bn; }
  }
  // hidden_drain: only tiles whose drain hides behind the next tile's K loop (the drain stores over NVLink)
  if (!hidden_drain) {
    const long t1 = rows256 * ((m_tok + 255) / 256);
    const double crowd = t1 <= pairs ? 0.85 : 1.0;     // one, partly filled pass: measured 46 us on 4096 x 11008 at 1024 tokens
    const double c = 8.5 + waves(t1) * (k128 * (0.159 + 0.00102 * 256) * f12 * crowd + (swiglu ? 2.0 : 4.0));
    if (c < best_cost * 0.97) { best_cost = c; best = 1256; }
  }
  if (!hidden_drain && m_tok >= 1024 && n_out >= 1024) {
    double c5 = 1e300;
    int b5 = 0;
    for (int bn : cands) {
      const long t2 = static_cast<long>((n_out + 511) / 512) * ((m_tok + bn - 1) / bn);
      const double crowd = t2 <= pairs ? 0.93 : 1.0;   // a single, partly filled pass: less contention for L2 (measured)
      const double c = 8.5 + waves(t2) * (k128 * (0.247 + 0.00199 * bn) * crowd + (swiglu ? 1.5 : 4.0));
      if (c < c5 * 0.985) { c5 = c; b5 = 5000 + bn; }
    }
    if (c5 < best_cost * 0.98) { best_cost = c5; best = b5; }
  }
  if (cost_us) *cost_us = best_cost;
  return best;
}

template <int EPI>
int dispatch_pair(const SparseGemmArgs& a, cudaStream_t stream) {
  // force_bn: 1256 / 1240 / 1224 / 1208 / 1192 = 256-row tiles with that many tokens;
  // 2192 / 2208 / 2224 / 2240 = 512-row tiles with that many tokens.  0 = automatic.
  int v = a.force_bn;
  if (v == 0) v = pick_pair_variant_impl(a.n_out, a.m_tok, a.K, a.num_sms / 2, EPI == kEpiSwiGLU, nullptr, a.peer_y != nullptr);
  switch (v) {
    case 1256: return launch_pair_cfg<PairCfg<256, 128, 4, 1, EPI>>(a, stream);
    case 1240: return launch_pair_cfg<PairCfg<240, 128, 4, 1, EPI>>(a, stream);
    case 1224: return launch_pair_cfg<PairCfg<224, 128, 4, 1, EPI>>(a, stream);
    case 1208: return launch_pair_cfg<PairCfg<208, 128, 4, 1, EPI>>(a, stream);
    case 1192: return launch_pair_cfg<PairCfg<192, 128, 4, 1, EPI>>(a, stream);
    case 5240: return launch_pair_cfg<PairCfg<240, 128, 3, 2, EPI>>(a, stream);
    case 5224: return launch_pair_cfg<PairCfg<224, 128, 3, 2, EPI>>(a, stream);
    case 5208: return launch_pair_cfg<PairCfg<208, 128, 3, 2, EPI>>(a, stream);
    case 5192: return launch_pair_cfg<PairCfg<192, 128, 3, 2, EPI>>(a, stream);
    case 2192: return launch_pair_cfg<PairCfg<192, 64, 6, 2, EPI>>(a, stream);
    case 2208: return launch_pair_cfg<PairCfg<208, 64, 6, 2, EPI>>(a, stream);
    case 2224: return launch_pair_cfg<PairCfg<224, 64, 6, 2, EPI>>(a, stream);
    case 2240: return launch_pair_cfg<PairCfg<240, 64, 6, 2, EPI>>(a, stream);
    default: return kErrInvalid;
  }
}

}  // namespace

void set_pair_tuning(int l2_band_mb, int force_order) {
  if (l2_band_mb > 0) g_l2_band_mb = l2_band_mb;
  g_force_order = force_order;
}

int pick_pair_variant(int n_out, int m_tok, int K, int num_sms, int swiglu, double* cost_us) {
  return pick_pair_variant_impl(n_out, m_tok, K, num_sms / 2 > 0 ? num_sms / 2 : 1, swiglu, cost_us);
}

int launch_sparse_gemm_pair(const SparseGemmArgs& a, cudaStream_t stream) {
  if (a.K % 64 != 0 || a.K <= 0 || a.m_tok <= 0 || a.n_out <= 0) return kErrInvalid;
  if (a.n_out % 8 != 0 || a.ldx % 8 != 0) return kErrInvalid;
  if ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.values) |
       reinterpret_cast<uintptr_t>(a.meta) | reinterpret_cast<uintptr_t>(a.y)) & 15)
    return kErrInvalid;
  if (a.ldy % 8 != 0) return kErrInvalid;
  if ((a.out_f32 || a.peer_y != nullptr) && a.epi != kEpiStore) return kErrInvalid;
  if (a.y == nullptr && a.peer_y == nullptr) return kErrInvalid;
  if (a.epi == kEpiSwiGLU) {
    if (a.n_out % 32 != 0 || (a.n_out / 2) % 8 != 0) return kErrInvalid;
    return dispatch_pair<kEpiSwiGLU>(a, stream);
  }
  return dispatch_pair<kEpiStore>(a, stream);
}

}  // namespace sfb200
