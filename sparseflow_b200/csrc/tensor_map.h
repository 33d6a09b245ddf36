// Host-side TMA tensor-map encoding (driver entry point resolved at run time, no libcuda link).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace sfb200 {

// 2-D row-major tensor of 16-bit elements [rows, cols] with row pitch `pitch_bytes`;
// box = box_rows x box_cols.  fmt: 0 = f16, 1 = bf16.
bool make_map_2d(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                 uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle sw, int fmt);
// 1-D tensor of 64-bit words.
bool make_map_1d_u64(CUtensorMap* m, const void* base, uint64_t elems, uint32_t box);

}  // namespace sfb200
