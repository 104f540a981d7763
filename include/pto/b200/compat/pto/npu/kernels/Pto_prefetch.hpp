// PTO_PREFETCH of the reference (include/pto/npu/kernels/Pto_prefetch.hpp:78-96) warms the NPU's L2 with a tensor before
// a kernel starts, by SDMA or by a kernel on the vector cores.  B200's L2 is filled by the kernel's own loads; the call
// is accepted and does nothing.
#pragma once
#include <cstddef>

template <bool UseSdma = true, int AivCores = -1>
inline void PTO_PREFETCH(void *tensor, std::size_t bytes, void *stream)
{
    (void)tensor;
    (void)bytes;
    (void)stream;
}
