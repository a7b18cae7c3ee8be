// One family of the tcgen05 GEMM kernel (see gemm_tc.cuh): <operand bytes, output type, fused epilogue> = <2, TVK_BF16, false>.
#include "gemm_tc.cuh"

namespace tvk {
namespace tc {

int launch_bf16(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s) { return launch_family<2, TVK_BF16, false>(bn, mt, maps, p, s); }

}  // namespace tc
}  // namespace tvk
