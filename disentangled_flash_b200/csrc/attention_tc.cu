// placeholder until the tcgen05 attention kernel lands
#include "dfl_common.cuh"
namespace dfl {
int launch_attention_tc(const DflAttnParams&, cudaStream_t) { return fail(DFL_ERR_UNSUPPORTED, "tcgen05 attention not built"); }
}
