// Exports the symbol the reference's GEMM ctypes loader binds: `call_kernel(blockDim, stream, out, src0, src1)`
// (demos/torch_jit/gemm/gemm_kernel.cpp:259-262), forwarding to the B200 kernel in libpto_b200.so.
#include "../../include/pto_b200.h"

extern "C" void call_kernel(uint32_t blockDim, void *stream, uint8_t *out, uint8_t *src0, uint8_t *src1)
{
    pto_b200_gemm_call_kernel(blockDim, stream, out, src0, src1);
}
