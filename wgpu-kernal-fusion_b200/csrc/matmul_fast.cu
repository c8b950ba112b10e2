#include "matmul.hpp"

namespace wgf {

bool matmul_fast_path(Device&, const void*, const void*, void*, DType, const MatmulDims&) { return false; }

}  // namespace wgf
