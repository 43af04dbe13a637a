// Tensor-core hashed attention for 16-bit inputs (placeholder dispatch until the kernel lands).
#include "attn_common.cuh"

namespace fm {

bool attn_mma_supported(int dtype, int d)
{
    (void)dtype;
    (void)d;
    return false;
}

int launch_attn_mma(const AttnParams &p, int dtype, int d, int grid, cudaStream_t st)
{
    (void)p; (void)dtype; (void)d; (void)grid; (void)st;
    set_error("tensor-core attention kernel not built for this shape");
    return FM_ERR_UNSUPPORTED;
}

}  // namespace fm
