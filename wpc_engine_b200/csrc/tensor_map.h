// TMA descriptors of row-major bfloat16 matrices, shared by the kernels that copy with TMA.
#pragma once
#include <cuda.h>

namespace wpc {
namespace tc {

// A tensor map for a row-major bfloat16 matrix [rows, cols] with row stride ld elements, copied
// in boxes of box_rows x 64 elements with the 128-byte swizzle (defined in gemm_tc.cu; encoded
// maps are kept, keyed by all arguments).  Returns 0 or a WPC_ERR_* code.
int tensor_map(const void* ptr, int rows, int cols, int ld, int box_rows, CUtensorMap* out);

}  // namespace tc
}  // namespace wpc
