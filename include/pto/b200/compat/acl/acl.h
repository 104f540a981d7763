// The few names of the Ascend runtime header that the reference's kernel files use in their launcher signatures
// (kernels/manual/common/flash_atten/fa_performance_kernel.cpp:972-1040 in the reference: aclFloat16 operands and an
// aclrtStream).  Hosts on B200 use the CUDA runtime; this header only lets those kernel files compile as they are.
// Add include/pto/b200/compat to the include path after include/.
#pragma once
#include <cuda_fp16.h>

typedef __half aclFloat16;
typedef void *aclrtStream;
