// Host-side helpers shared by the C-ABI entry points: TMA descriptor encoding through the
// driver entry point (no link-time dependency on libcuda) and cached device properties.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "../../include/msl.h"

namespace msl {

int sm_count();

// 2-D tensor map over a row-major matrix: `cols` elements per row (innermost), `rows` rows,
// `row_pitch_bytes` between rows; the box is box_cols x box_rows elements.
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t cols,
                 uint64_t rows, uint64_t row_pitch_bytes, uint32_t box_cols, uint32_t box_rows,
                 CUtensorMapSwizzle swizzle);

// 3-D tensor map (innermost first): dims d0 x d1 x d2 with byte pitches p1 (between d1 steps)
// and p2 (between d2 steps); box b0 x b1 x b2.
int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, uint64_t d0, uint64_t d1,
                 uint64_t d2, uint64_t p1, uint64_t p2, uint32_t b0, uint32_t b1, uint32_t b2,
                 CUtensorMapSwizzle swizzle);

}  // namespace msl
