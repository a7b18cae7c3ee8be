// One family of the tcgen05 GEMM kernel (see gemm_tc.cuh): <operand bytes, output type, fused epilogue> = <4, TVK_F32, false>.
#include "gemm_tc.cuh"

namespace tvk {
namespace tc {

int launch_tf32(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s) { return launch_family<4, TVK_F32, false>(bn, mt, maps, p, s); }

}  // namespace tc
}  // namespace tvk
