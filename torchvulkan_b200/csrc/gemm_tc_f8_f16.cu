// The tcgen05 GEMM kernel for float8 operands (tcgen05.mma kind::f8f6f4) with a f16 result: the scaled product with its
// scales, bias and cast applied by the epilogue (see gemm_tc.cuh, Params::row_scale / col_scale).
#include "gemm_tc.cuh"

namespace tvk {
namespace tc {

int launch_f8_f16out(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s) { return launch_family<1, TVK_F16, false>(bn, mt, maps, p, s); }

}  // namespace tc
}  // namespace tvk
