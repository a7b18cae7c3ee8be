// One family of the tcgen05 GEMM kernel (see gemm_tc.cuh): <operand bytes, output type, fused epilogue> = <2, TVK_F32, false>.
#include "gemm_tc.cuh"

namespace tvk {
namespace tc {

int launch_half_f32out(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s) { return launch_family<2, TVK_F32, false>(bn, mt, maps, p, s); }

}  // namespace tc
}  // namespace tvk
