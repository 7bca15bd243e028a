// tcgen05 prefill instance (placeholder until the kernel lands): reports "not supported" so that the
// dispatcher uses the general instance.
#include <string.h>

#include "kernels.h"

namespace fck {
bool fwd_sm100_supported(const FwdParams&) { return false; }
int launch_fwd_sm100(const FwdParams&, cudaStream_t) {
    set_last_error("fmha_fwd: the tcgen05 instance is not built");
    return FLASHCK_ERR_UNSUPPORTED;
}
int fwd_set_param(const char*, int64_t) { return FLASHCK_ERR_INVALID_ARGUMENT; }
int fwd_get_param(const char*, int64_t*) { return FLASHCK_ERR_INVALID_ARGUMENT; }
}  // namespace fck
