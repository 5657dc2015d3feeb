// placeholder until the tcgen05 GEMM lands
#include "dfl_common.cuh"
namespace dfl {
int launch_gemm_tc(const GemmDesc&, cudaStream_t) { return fail(DFL_ERR_UNSUPPORTED, "tcgen05 GEMM not built"); }
}
