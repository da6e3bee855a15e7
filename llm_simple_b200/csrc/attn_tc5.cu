// placeholder until the tcgen05 kernel lands
#include "kernels.h"
namespace b200attn {
cudaError_t launch_attn_prefill_tc5(const PrefillParams &, bool, cudaStream_t) { return cudaErrorNotSupported; }
}
