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
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace sfb200 {
namespace {

constexpr uint32_t kPadNibble = 0x4;
constexpr uint32_t kPadMeta16 = 0x4444;
// nibble (idx0 | idx1<<2) -> reference code byte
constexpr unsigned long long kRefCodeLut = (9ull << 16) | (4ull << 32) | (8ull << 48) |
                                           (12ull << 36) | (14ull << 52) | (13ull << 56);

struct GroupOut {
  uint32_t vals;    // kept pair, low half first
  uint32_t nib;     // idx0 | idx1 << 2
  uint32_t lo, hi;  // pruned group
};

// lo = (e0, e1), hi = (e2, e3) as 16-bit patterns; nan_clamp = inf pattern + 1.
// Key = (min(|w| pattern, nan_clamp) << 2) | tie bits, unique within the group, so the two kept
// elements are the two largest keys and their positions are the keys' low two bits.  A five
// comparator network finds them: (a,b) = sort(k0,k1), (c,d) = sort(k2,k3); largest = max(b,d),
// second = max(min(b,d), max(a,c)).
template <int TIE>
__device__ __forceinline__ GroupOut select_group(uint32_t lo, uint32_t hi, uint32_t nan_clamp) {
  uint32_t k0 = min(lo & 0x7FFFu, nan_clamp), k1 = min((lo >> 16) & 0x7FFFu, nan_clamp);
  uint32_t k2 = min(hi & 0x7FFFu, nan_clamp), k3 = min((hi >> 16) & 0x7FFFu, nan_clamp);
  if (TIE == kTieHigh) {
    k0 = k0 * 4 + 0; k1 = k1 * 4 + 1; k2 = k2 * 4 + 2; k3 = k3 * 4 + 3;
  } else {
    k0 = k0 * 4 + 3; k1 = k1 * 4 + 2; k2 = k2 * 4 + 1; k3 = k3 * 4 + 0;
  }
  const uint32_t a = min(k0, k1), b = max(k0, k1), c = min(k2, k3), d = max(k2, k3);
  const uint32_t first = max(b, d);
  const uint32_t second = max(min(b, d), max(a, c));
  uint32_t pa = first & 3u, pb = second & 3u;
  if (TIE == kTieLow) { pa = 3u - pa; pb = 3u - pb; }
  const uint32_t i0 = min(pa, pb), i1 = max(pa, pb);
  GroupOut o;
  o.nib = i0 | (i1 << 2);
  // byte selectors (2*i, 2*i+1) for both kept elements
  const uint32_t sel = (i0 * 0x22u + 0x10u) | ((i1 * 0x22u + 0x10u) << 8);
  o.vals = __byte_perm(lo, hi, sel);
  const uint32_t mask = (1u << i0) | (1u << i1);
  o.lo = lo & ((mask & 1 ? 0xFFFFu : 0u) | (mask & 2 ? 0xFFFF0000u : 0u));
  o.hi = hi & ((mask & 4 ? 0xFFFFu : 0u) | (mask & 8 ? 0xFFFF0000u : 0u));
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
  uint32_t nan_clamp;
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
__device__ __forceinline__ uint32_t process_row16(const PruneParams& p, int r, int k0) {
  if (r >= p.out_rows || k0 >= p.K) return kPadMeta16;
  const uint4* s = reinterpret_cast<const uint4*>(src_row(p, r) + k0);
  const uint4 a = __ldg(s), b = __ldg(s + 1);
  const GroupOut g0 = select_group<TIE>(a.x, a.y, p.nan_clamp);
  const GroupOut g1 = select_group<TIE>(a.z, a.w, p.nan_clamp);
  const GroupOut g2 = select_group<TIE>(b.x, b.y, p.nan_clamp);
  const GroupOut g3 = select_group<TIE>(b.z, b.w, p.nan_clamp);
  if (p.values) {
    uint4 v = make_uint4(g0.vals, g1.vals, g2.vals, g3.vals);
    *reinterpret_cast<uint4*>(p.values + static_cast<size_t>(r) * (p.K / 2) + k0 / 2) = v;
  }
  if (p.pruned) {
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
  return g0.nib | (g1.nib << 4) | (g2.nib << 8) | (g3.nib << 12);
}

// grid: (ceil(Kpad / 512), Rpad / 16), block 256: warp w -> rows m0 = w and w + 8 of the 16-row
// group, lane -> 16-element K slice.
template <int TIE>
__global__ void __launch_bounds__(256) prune_compress_kernel(const PruneParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = (blockIdx.x * 32 + lane) * 16;
  if (k0 >= p.k_tiles128 * 128) return;
  const int r_a = blockIdx.y * 16 + warp;
  const uint32_t ma = process_row16<TIE>(p, r_a, k0);
  const uint32_t mb = process_row16<TIE>(p, r_a + 8, k0);
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
  const int G = p.K / 4;
  const size_t total = static_cast<size_t>(p.out_rows) * G;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / G), g = static_cast<int>(i % G);
    const uint2 v = *reinterpret_cast<const uint2*>(src_row(p, r) + 4 * g);
    const GroupOut o = select_group<TIE>(v.x, v.y, p.nan_clamp);
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
  p.nan_clamp = (a.fmt == kF16 ? 0x7C00u : 0x7F80u) + 1;
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
