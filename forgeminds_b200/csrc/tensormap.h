// Host-side construction (and caching) of TMA tensor maps. The driver entry point is resolved at
// run time through the CUDA runtime, so the library does not link against libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmb {

enum class TmapSwizzle : int { None = 0, B32 = 1, B64 = 2, B128 = 3 };

// 2-D row-major tensor [rows, cols] of `elem_bytes`-sized elements with row pitch `ld` elements,
// copied in boxes of [box_rows, box_cols]. Returns false (and leaves `out` untouched) on failure.
bool make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                  uint32_t box_rows, uint32_t box_cols, int elem_bytes, TmapSwizzle swz);

// General N-d (<= 5) variant: dims/strides innermost first; strides[0] is implied (elem_bytes).
bool make_tmap_nd(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                  const uint64_t* strides_bytes, const uint32_t* box, int elem_bytes, TmapSwizzle swz);

int sm_count();

}  // namespace fmb
