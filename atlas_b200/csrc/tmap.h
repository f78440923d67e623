// Tensor-map construction shared by the GEMM translation units (implemented in gemm.cu, cached by key).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace atlas {
// Row-major [rows, cols] matrix of `esize`-byte elements with leading dimension `ld` (elements); tiles of
// box_rows x box_bytes.  swizzle128 selects CU_TENSOR_MAP_SWIZZLE_128B (box_bytes must then be 128), otherwise the
// tile lands row after row without swizzling.  Returns 0 or a negative error code.
int make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                 uint32_t esize, uint32_t box_bytes, bool swizzle128);
}  // namespace atlas
