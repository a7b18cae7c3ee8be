// The tcgen05 GEMM kernel for float8 operands (e4m3 / e5m2, tcgen05.mma kind::f8f6f4) with an fp32 result: the product
// behind _scaled_mm (scaled_mm.cu applies the scales, the bias and the cast to the accumulator it leaves).
#include "gemm_tc.cuh"

namespace tvk {
namespace tc {

int launch_f8_f32out(int bn, int mt, const CUtensorMap* maps, const Params& p, cudaStream_t s) { return launch_family<1, TVK_F32, false>(bn, mt, maps, p, s); }

}  // namespace tc
}  // namespace tvk
