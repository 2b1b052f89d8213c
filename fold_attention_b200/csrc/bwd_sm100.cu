// placeholder until the tcgen05 kernel lands
#include "bwd_common.cuh"
namespace fold {
bool bwd_sm100_supported(const BwdParams&) { return false; }
int launch_bwd_main_sm100(const BwdParams&, cudaStream_t) {
    set_error("the tcgen05 backward is not built");
    return FOLD_ERR_UNSUPPORTED;
}
}  // namespace fold
