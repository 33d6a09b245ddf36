// Standalone SiLU.mul: out = (g * 1/(1+exp(-g))) * u in fp32, stored in the 16-bit type.
// Same arithmetic as the reference's Triton kernel (sparseflow/kernels/fused_silu_mul.py:6-31);
// used on the dense branch of the shape gate and as the unfused A/B variant of the fused epilogue.
// HBM-bound: 3 x 2 bytes per element; 16-byte vector accesses, grid sized to the SM count.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace sfb200 {
namespace {

template <bool BF16>
__device__ __forceinline__ float ld16(uint16_t b) {
  if (BF16) return __uint_as_float(static_cast<uint32_t>(b) << 16);
  return __half2float(__ushort_as_half(b));
}
template <bool BF16>
__device__ __forceinline__ uint16_t st16(float v) {
  if (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  return __half_as_ushort(__float2half_rn(v));
}
template <bool BF16>
__device__ __forceinline__ uint32_t silu_mul2(uint32_t g2, uint32_t u2) {
  uint32_t r = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float g = ld16<BF16>(static_cast<uint16_t>(g2 >> (16 * h)));
    const float u = ld16<BF16>(static_cast<uint16_t>(u2 >> (16 * h)));
    const float s = 1.0f / (1.0f + __expf(-g));
    r |= static_cast<uint32_t>(st16<BF16>((g * s) * u)) << (16 * h);
  }
  return r;
}

// vec path: cols % 8 == 0, all pitches % 8 == 0, 16-byte aligned bases
template <bool BF16>
__global__ void __launch_bounds__(256) silu_mul_vec_kernel(const uint16_t* g, const uint16_t* u,
                                                           uint16_t* o, int rows, int cols, int ldg,
                                                           int ldu, int ldo) {
  const int vcols = cols / 8;
  const size_t total = static_cast<size_t>(rows) * vcols;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / vcols), c = static_cast<int>(i % vcols) * 8;
    const uint4 gv = __ldg(reinterpret_cast<const uint4*>(g + static_cast<size_t>(r) * ldg + c));
    const uint4 uv = __ldg(reinterpret_cast<const uint4*>(u + static_cast<size_t>(r) * ldu + c));
    uint4 ov;
    ov.x = silu_mul2<BF16>(gv.x, uv.x);
    ov.y = silu_mul2<BF16>(gv.y, uv.y);
    ov.z = silu_mul2<BF16>(gv.z, uv.z);
    ov.w = silu_mul2<BF16>(gv.w, uv.w);
    *reinterpret_cast<uint4*>(o + static_cast<size_t>(r) * ldo + c) = ov;
  }
}

template <bool BF16>
__global__ void silu_mul_scalar_kernel(const uint16_t* g, const uint16_t* u, uint16_t* o, int rows,
                                       int cols, int ldg, int ldu, int ldo) {
  const size_t total = static_cast<size_t>(rows) * cols;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / cols), c = static_cast<int>(i % cols);
    const float gv = ld16<BF16>(g[static_cast<size_t>(r) * ldg + c]);
    const float uv = ld16<BF16>(u[static_cast<size_t>(r) * ldu + c]);
    const float s = 1.0f / (1.0f + __expf(-gv));
    o[static_cast<size_t>(r) * ldo + c] = st16<BF16>((gv * s) * uv);
  }
}

}  // namespace

int launch_silu_mul(const void* gate, const void* up, void* out, int rows, int cols, int ld_g,
                    int ld_u, int ld_o, int fmt, cudaStream_t stream) {
  if (!gate || !up || !out || rows <= 0 || cols <= 0) return kErrInvalid;
  if (ld_g < cols || ld_u < cols || ld_o < cols) return kErrInvalid;
  if (fmt != kF16 && fmt != kBF16) return kErrInvalid;
  const uint16_t* g = static_cast<const uint16_t*>(gate);
  const uint16_t* u = static_cast<const uint16_t*>(up);
  uint16_t* o = static_cast<uint16_t*>(out);
  const bool vec = cols % 8 == 0 && ld_g % 8 == 0 && ld_u % 8 == 0 && ld_o % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                     reinterpret_cast<uintptr_t>(out)) % 16 == 0);
  const size_t work = vec ? static_cast<size_t>(rows) * (cols / 8) : static_cast<size_t>(rows) * cols;
  size_t blocks = (work + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (vec) {
    if (fmt == kBF16) silu_mul_vec_kernel<true><<<blocks, 256, 0, stream>>>(g, u, o, rows, cols, ld_g, ld_u, ld_o);
    else silu_mul_vec_kernel<false><<<blocks, 256, 0, stream>>>(g, u, o, rows, cols, ld_g, ld_u, ld_o);
  } else {
    if (fmt == kBF16) silu_mul_scalar_kernel<true><<<blocks, 256, 0, stream>>>(g, u, o, rows, cols, ld_g, ld_u, ld_o);
    else silu_mul_scalar_kernel<false><<<blocks, 256, 0, stream>>>(g, u, o, rows, cols, ld_g, ld_u, ld_o);
  }
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}

}  // namespace sfb200
