// 2:4 magnitude prune + compress, bit-exact with the reference CPU path
// (experiments/prune_24_cpu.py:17-28): per row, per group of four along K keep the two entries
// with the largest |w|; ties go to the higher index (tie mode "high", the script's behaviour) or
// the lower index (tie mode "low"); NaN ranks above everything; -0 == +0.
//
// Outputs (each optional):
//   values    [rows, K/2]  kept entries in index order                  (script: dA.bin)
//   ref_codes [rows, K/4]  one byte per group, PAIR_TO_CODE table       (script: dE.bin, :12-15)
//   pruned    [rows, K]    kept entries in place, +0 elsewhere          (script: A_pruned_dense.bin)
//   meta      tiled 2-bit metadata in the layout tcgen05.mma.sp reads from tensor memory:
//     tile = 128 rows x 128 logical K = 128 lanes x 4 uint32 (2 KiB contiguous), tiles ordered
//     [row_tile][k_tile].  For row m = m0 + 8*m1 + 16*m2, 32-wide K block kb, 16-wide half kh:
//     lane = m0 + 8*kh + 16*m2, word = kb, bits [16*m1, 16*m1+16) = 4 nibbles (group j at 4j),
//     nibble = idx0 | idx1 << 2.  Rows / K beyond the matrix are filled with nibble 0x4.
//
// HBM-bound: 2 B read + 1 B values + 1/8 B metadata per weight element.  One thread owns 16
// consecutive K elements of rows m and m+8 (two 16-byte loads per row), which is exactly one
// 32-bit metadata word; a warp streams 1 KiB of each of its two rows.
//
// Selection, two groups at a time in packed 16-bit halves (the integer pipe, not HBM, bounded the earlier
// one-group-at-a-time forms: pairwise ranking ~95 instructions per group, 34 % of HBM; a key-sorting network of
// five comparators ~50, 59 %): the magnitudes m_i of element i of both groups sit in the two halves of one word,
// a single subtraction per pair (i, j) decides "j beats i" for both groups (bit 15 of each half of
// (m_j | 0x8000) - m_i, no borrow crosses the halves), the six decision bits index a 64-entry table in shared
// memory that returns the kept pair as a metadata nibble and as the byte selector that gathers the two kept values.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace sfb200 {
namespace {

constexpr uint32_t kPadMeta16 = 0x4444;
// nibble (idx0 | idx1<<2) -> reference code byte
constexpr unsigned long long kRefCodeLut = (9ull << 16) | (4ull << 32) | (8ull << 48) |
                                           (12ull << 36) | (14ull << 52) | (13ull << 56);

struct GroupOut {
  uint32_t vals;    // kept pair, low half first
  uint32_t nib;     // idx0 | idx1 << 2
  uint32_t lo, hi;  // pruned group
};

// Table: decision bits (b01, b02, b03, b12, b13, b23) at bit 0..5, b_ij = "element j beats element i" (i < j)
// -> byte selector of the kept pair in bits [0, 16) (bytes 2*i0, 2*i0+1, 2*i1, 2*i1+1 of the group's two words)
// and the nibble idx0 | idx1 << 2 in bits [16, 20).  An element is kept when at most one other element beats it.
struct SelectLut {
  uint32_t e[64];
};
constexpr SelectLut make_select_lut() {
  SelectLut t{};
  for (int p = 0; p < 64; ++p) {
    const int b01 = p & 1, b02 = (p >> 1) & 1, b03 = (p >> 2) & 1, b12 = (p >> 3) & 1, b13 = (p >> 4) & 1, b23 = (p >> 5) & 1;
    const int beaten[4] = {b01 + b02 + b03, (1 - b01) + b12 + b13, (1 - b02) + (1 - b12) + b23,
                           (1 - b03) + (1 - b13) + (1 - b23)};
    int i0 = -1, i1 = -1;
    for (int i = 0; i < 4; ++i)
      if (beaten[i] <= 1) {
        if (i0 < 0) i0 = i;
        else if (i1 < 0) i1 = i;
      }
    if (i1 < 0) { i0 = 0; i1 = 1; }   // intransitive patterns: cannot come out of a total order
    const uint32_t sel = static_cast<uint32_t>((2 * i0) | ((2 * i0 + 1) << 4) | ((2 * i1) << 8) | ((2 * i1 + 1) << 12));
    t.e[p] = sel | (static_cast<uint32_t>(i0 | (i1 << 2)) << 16);
  }
  return t;
}
__device__ const SelectLut kSelectLut = make_select_lut();

__device__ __forceinline__ uint32_t min_u16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("min.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Two groups at once: (lo0, hi0) and (lo1, hi1), each lo = (e0, e1), hi = (e2, e3) as 16-bit patterns.
// clamp2 = (inf pattern + 1) in both halves: every NaN becomes the same largest magnitude, so NaNs tie.
// TIE high: j beats i (i < j) iff m_j >= m_i;  TIE low: iff m_j > m_i.  Returns the two table entries.
template <int TIE>
__device__ __forceinline__ void select_pair(uint32_t lo0, uint32_t hi0, uint32_t lo1, uint32_t hi1, uint32_t clamp2,
                                            const uint32_t* lut, uint32_t& e0, uint32_t& e1) {
  // element i of both groups side by side
  const uint32_t m0 = min_u16x2(__byte_perm(lo0, lo1, 0x5410) & 0x7FFF7FFFu, clamp2);
  const uint32_t m1 = min_u16x2(__byte_perm(lo0, lo1, 0x7632) & 0x7FFF7FFFu, clamp2);
  const uint32_t m2 = min_u16x2(__byte_perm(hi0, hi1, 0x5410) & 0x7FFF7FFFu, clamp2);
  const uint32_t m3 = min_u16x2(__byte_perm(hi0, hi1, 0x7632) & 0x7FFF7FFFu, clamp2);
  // bit 15 of each half of (m_j | 0x8000) - m_i (- 1 for "strictly greater") = "j beats i"; magnitudes are below
  // 0x8000, so no half borrows from the other
  constexpr uint32_t kBias = (TIE == kTieHigh) ? 0x80008000u : 0x7FFF7FFFu;
  const uint32_t q1 = m1 + kBias, q2 = m2 + kBias, q3 = m3 + kBias;
  const uint32_t d01 = q1 - m0, d02 = q2 - m0, d03 = q3 - m0, d12 = q2 - m1, d13 = q3 - m1, d23 = q3 - m2;
  const uint32_t idx = ((d01 >> 15) & 0x00010001u) | ((d02 >> 14) & 0x00020002u) | ((d03 >> 13) & 0x00040004u) |
                       ((d12 >> 12) & 0x00080008u) | ((d13 >> 11) & 0x00100010u) | ((d23 >> 10) & 0x00200020u);
  e0 = lut[idx & 0x3Fu];
  e1 = lut[idx >> 16];
}

__device__ __forceinline__ GroupOut finish_group(uint32_t lo, uint32_t hi, uint32_t entry, bool want_pruned) {
  GroupOut o;
  o.vals = __byte_perm(lo, hi, entry);      // the selector is the entry's low 16 bits
  o.nib = entry >> 16;
  o.lo = o.hi = 0;
  if (want_pruned) {
    const uint32_t i0 = o.nib & 3u, i1 = o.nib >> 2;
    const uint32_t mask = (1u << i0) | (1u << i1);
    o.lo = lo & ((mask & 1 ? 0xFFFFu : 0u) | (mask & 2 ? 0xFFFF0000u : 0u));
    o.hi = hi & ((mask & 4 ? 0xFFFFu : 0u) | (mask & 8 ? 0xFFFF0000u : 0u));
  }
  return o;
}

struct PruneParams {
  const uint16_t* src0;
  const uint16_t* src1;
  uint16_t* values;
  uint32_t* meta;
  uint8_t* ref_codes;
  uint16_t* pruned;
  int out_rows, K, ld, interleave;
  int k_tiles128;
  uint32_t clamp2;     // (inf pattern + 1) in both 16-bit halves
};

__device__ __forceinline__ const uint16_t* src_row(const PruneParams& p, int r) {
  if (p.interleave == 0) return p.src0 + static_cast<size_t>(r) * p.ld;
  const int B = p.interleave;
  const int blk = r / (2 * B), w = r % (2 * B);
  const uint16_t* base = (w < B) ? p.src0 : p.src1;
  return base + static_cast<size_t>(blk * B + (w % B)) * p.ld;
}

// Processes 16 elements of one row; returns the 16-bit metadata half word.
template <int TIE>
__device__ __forceinline__ uint32_t process_row16(const PruneParams& p, const uint32_t* lut, int r, int k0) {
  if (r >= p.out_rows || k0 >= p.K) return kPadMeta16;
  const uint4* s = reinterpret_cast<const uint4*>(src_row(p, r) + k0);
  const uint4 a = __ldg(s), b = __ldg(s + 1);
  uint32_t e0, e1, e2, e3;
  select_pair<TIE>(a.x, a.y, a.z, a.w, p.clamp2, lut, e0, e1);
  select_pair<TIE>(b.x, b.y, b.z, b.w, p.clamp2, lut, e2, e3);
  const bool want_pruned = p.pruned != nullptr;
  const GroupOut g0 = finish_group(a.x, a.y, e0, want_pruned), g1 = finish_group(a.z, a.w, e1, want_pruned);
  const GroupOut g2 = finish_group(b.x, b.y, e2, want_pruned), g3 = finish_group(b.z, b.w, e3, want_pruned);
  if (p.values) {
    uint4 v = make_uint4(g0.vals, g1.vals, g2.vals, g3.vals);
    *reinterpret_cast<uint4*>(p.values + static_cast<size_t>(r) * (p.K / 2) + k0 / 2) = v;
  }
  if (want_pruned) {
    uint4* d = reinterpret_cast<uint4*>(p.pruned + static_cast<size_t>(r) * p.K + k0);
    d[0] = make_uint4(g0.lo, g0.hi, g1.lo, g1.hi);
    d[1] = make_uint4(g2.lo, g2.hi, g3.lo, g3.hi);
  }
  if (p.ref_codes) {
    const uint32_t c = static_cast<uint32_t>((kRefCodeLut >> (4 * g0.nib)) & 0xF) |
                       static_cast<uint32_t>((kRefCodeLut >> (4 * g1.nib)) & 0xF) << 8 |
                       static_cast<uint32_t>((kRefCodeLut >> (4 * g2.nib)) & 0xF) << 16 |
                       static_cast<uint32_t>((kRefCodeLut >> (4 * g3.nib)) & 0xF) << 24;
    *reinterpret_cast<uint32_t*>(p.ref_codes + static_cast<size_t>(r) * (p.K / 4) + k0 / 4) = c;
  }
  return (e0 >> 16) | ((e1 >> 12) & 0xF0u) | ((e2 >> 8) & 0xF00u) | ((e3 >> 4) & 0xF000u);
}

// grid: (ceil(Kpad / 512), Rpad / 16), block 256: warp w -> rows m0 = w and w + 8 of the 16-row
// group, lane -> 16-element K slice.
template <int TIE>
__global__ void __launch_bounds__(256) prune_compress_kernel(const PruneParams p) {
  __shared__ uint32_t lut[64];
  if (threadIdx.x < 64) lut[threadIdx.x] = kSelectLut.e[threadIdx.x];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = (blockIdx.x * 32 + lane) * 16;
  if (k0 >= p.k_tiles128 * 128) return;
  const int r_a = blockIdx.y * 16 + warp;
  const uint32_t ma = process_row16<TIE>(p, lut, r_a, k0);
  const uint32_t mb = process_row16<TIE>(p, lut, r_a + 8, k0);
  if (p.meta) {
    const int rt = r_a >> 7, m2 = (r_a & 127) >> 4;
    const int kt = k0 >> 7, kb = (k0 & 127) >> 5, kh = (k0 & 31) >> 4;
    const int ln = warp + 8 * kh + 16 * m2;
    p.meta[((static_cast<size_t>(rt) * p.k_tiles128 + kt) * 128 + ln) * 4 + kb] = ma | (mb << 16);
  }
}

// Any K % 4 == 0: one thread per group, no tiled metadata.
template <int TIE>
__global__ void prune_generic_kernel(const PruneParams p) {
  __shared__ uint32_t lut[64];
  if (threadIdx.x < 64) lut[threadIdx.x] = kSelectLut.e[threadIdx.x];
  __syncthreads();
  const int G = p.K / 4;
  const size_t total = static_cast<size_t>(p.out_rows) * G;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / G), g = static_cast<int>(i % G);
    const uint2 v = *reinterpret_cast<const uint2*>(src_row(p, r) + 4 * g);
    uint32_t e0, e1;
    select_pair<TIE>(v.x, v.y, v.x, v.y, p.clamp2, lut, e0, e1);
    const GroupOut o = finish_group(v.x, v.y, e0, p.pruned != nullptr);
    if (p.values) *reinterpret_cast<uint32_t*>(p.values + static_cast<size_t>(r) * (p.K / 2) + 2 * g) = o.vals;
    if (p.pruned)
      *reinterpret_cast<uint2*>(p.pruned + static_cast<size_t>(r) * p.K + 4 * g) = make_uint2(o.lo, o.hi);
    if (p.ref_codes)
      p.ref_codes[static_cast<size_t>(r) * G + g] = static_cast<uint8_t>((kRefCodeLut >> (4 * o.nib)) & 0xF);
  }
}

__global__ void validate_24_kernel(const uint16_t* w, int rows, int K, int ld, int* flag) {
  const int G = K / 4;
  const size_t total = static_cast<size_t>(rows) * G;
  bool bad = false;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / G), g = static_cast<int>(i % G);
    const uint2 v = *reinterpret_cast<const uint2*>(w + static_cast<size_t>(r) * ld + 4 * g);
    const int nz = ((v.x & 0x7FFF) != 0) + ((v.x & 0x7FFF0000) != 0) + ((v.y & 0x7FFF) != 0) +
                   ((v.y & 0x7FFF0000) != 0);
    bad |= nz > 2;
  }
  if (bad) atomicExch(flag, 0);
}

__global__ void decompress_kernel(const uint16_t* values, const uint32_t* meta, int rows, int K,
                                  int k_tiles128, uint16_t* dense, int ld) {
  const int G = K / 4;
  const size_t total = static_cast<size_t>(rows) * G;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / G), g = static_cast<int>(i % G);
    const int k0 = 4 * g;
    const int rt = r >> 7, m = r & 127, m0 = m & 7, m1 = (m >> 3) & 1, m2 = m >> 4;
    const int kt = k0 >> 7, kb = (k0 & 127) >> 5, kh = (k0 & 31) >> 4, j = (k0 & 15) >> 2;
    const uint32_t word =
        meta[((static_cast<size_t>(rt) * k_tiles128 + kt) * 128 + (m0 + 8 * kh + 16 * m2)) * 4 + kb];
    const uint32_t nib = (word >> (16 * m1 + 4 * j)) & 0xF;
    const uint32_t pair = *reinterpret_cast<const uint32_t*>(values + static_cast<size_t>(r) * (K / 2) + 2 * g);
    uint16_t out[4] = {0, 0, 0, 0};
    out[nib & 3] = static_cast<uint16_t>(pair & 0xFFFF);
    out[(nib >> 2) & 3] = static_cast<uint16_t>(pair >> 16);
    uint16_t* d = dense + static_cast<size_t>(r) * ld + k0;
    *reinterpret_cast<uint2*>(d) = make_uint2(out[0] | (uint32_t(out[1]) << 16), out[2] | (uint32_t(out[3]) << 16));
  }
}

}  // namespace

int launch_prune_compress(const PruneArgs& a, cudaStream_t stream) {
  if (a.rows <= 0 || a.K <= 0 || a.K % 4 != 0 || a.dense == nullptr) return kErrInvalid;
  if (a.ld < a.K || a.ld % 4 != 0) return kErrInvalid;
  if (a.interleave != 0 && (a.dense2 == nullptr || a.interleave < 0 || a.rows % a.interleave != 0))
    return kErrInvalid;
  if (a.fmt != kF16 && a.fmt != kBF16) return kErrInvalid;
  PruneParams p;
  p.src0 = static_cast<const uint16_t*>(a.dense);
  p.src1 = static_cast<const uint16_t*>(a.dense2);
  p.values = static_cast<uint16_t*>(a.values);
  p.meta = static_cast<uint32_t*>(a.meta);
  p.ref_codes = static_cast<uint8_t*>(a.ref_codes);
  p.pruned = static_cast<uint16_t*>(a.pruned);
  p.out_rows = a.interleave ? 2 * a.rows : a.rows;
  p.K = a.K;
  p.ld = a.ld;
  p.interleave = a.interleave;
  p.k_tiles128 = (a.K + 127) / 128;
  p.clamp2 = ((a.fmt == kF16 ? 0x7C00u : 0x7F80u) + 1) * 0x00010001u;
  const bool vec_ok = (a.K % 16 == 0) && (a.ld % 8 == 0) &&
                      ((reinterpret_cast<uintptr_t>(a.dense) | reinterpret_cast<uintptr_t>(a.dense2) |
                        reinterpret_cast<uintptr_t>(a.values) | reinterpret_cast<uintptr_t>(a.pruned) |
                        reinterpret_cast<uintptr_t>(a.ref_codes)) % 16 == 0);
  if (vec_ok) {
    const int kpad = p.k_tiles128 * 128;
    const int rpad = ((p.out_rows + 127) / 128) * 128;
    dim3 grid((kpad + 511) / 512, rpad / 16);
    if (a.tie == kTieLow) prune_compress_kernel<kTieLow><<<grid, 256, 0, stream>>>(p);
    else prune_compress_kernel<kTieHigh><<<grid, 256, 0, stream>>>(p);
  } else {
    if (a.meta != nullptr) return kErrInvalid;  // tiled metadata needs K % 16 == 0 and 16-byte alignment
    if ((reinterpret_cast<uintptr_t>(a.dense) | reinterpret_cast<uintptr_t>(a.dense2)) % 8 != 0)
      return kErrInvalid;
    const size_t total = static_cast<size_t>(p.out_rows) * (a.K / 4);
    const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
    if (a.tie == kTieLow) prune_generic_kernel<kTieLow><<<blocks, 256, 0, stream>>>(p);
    else prune_generic_kernel<kTieHigh><<<blocks, 256, 0, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

int launch_validate_24(const void* w, int rows, int K, int ld, int* d_flag, cudaStream_t stream) {
  if (rows <= 0 || K <= 0 || K % 4 != 0 || ld % 4 != 0 || (reinterpret_cast<uintptr_t>(w) % 8) != 0)
    return kErrInvalid;
  const size_t total = static_cast<size_t>(rows) * (K / 4);
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  validate_24_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(w), rows, K, ld, d_flag);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

int launch_decompress(const void* values, const void* meta, int rows, int K, void* dense, int ld,
                      cudaStream_t stream) {
  if (rows <= 0 || K <= 0 || K % 4 != 0 || ld % 4 != 0) return kErrInvalid;
  const size_t total = static_cast<size_t>(rows) * (K / 4);
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  decompress_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(values),
                                                static_cast<const uint32_t*>(meta), rows, K,
                                                (K + 127) / 128, static_cast<uint16_t*>(dense), ld);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

}  // namespace sfb200
