#include "ptx.cuh"
#include "internal.h"
namespace pto_b200 {
int launch_flash_attn_fwd(const uint16_t *, const uint16_t *, const uint16_t *, void *, int, int, int, int, int, float,
                          int, cudaStream_t)
{
    set_error_text("flash attention: not built yet");
    return kErrUnsupportedShape;
}
} // namespace pto_b200
