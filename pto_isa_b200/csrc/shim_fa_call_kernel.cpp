// Exports the symbol the reference's flash-attention ctypes loader binds: `call_kernel(stream, headSize, s0, s1,
// is_causal, q, k, v, o_out, <seven workspaces>)` (demos/torch_jit/flash_atten/fa_kernel.cpp:1017-1037),
// forwarding to the B200 kernel in libpto_b200.so.
#include "../../include/pto_b200.h"

extern "C" void call_kernel(void *stream, int headSize, int s0, int s1, bool is_causal, uint8_t *q, uint8_t *k,
                            uint8_t *v, uint8_t *o_out, float *qk_ws, uint16_t *p_ws, float *pmax_ws, float *pv_ws,
                            float *gsum, float *expmax, float *o_parts)
{
    pto_b200_fa_call_kernel(stream, headSize, s0, s1, is_causal, q, k, v, o_out, qk_ws, p_ws, pmax_ws, pv_ws, gsum,
                            expmax, o_parts);
}
