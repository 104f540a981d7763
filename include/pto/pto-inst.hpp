// Entry header of the PTO tile ISA for the B200 (sm_100a) backend: `#include <pto/pto-inst.hpp>` and
// `using namespace pto;` as with the reference's header of the same name (include/pto/pto-inst.hpp:14-24 in the
// reference).  Compile with nvcc for sm_100a and `--extended-lambda`.
//
// Tile programs of the reference spell kernels `__global__ AICORE void f(...)` and, in its CPU-simulation
// style, call them like functions.  On this backend a tile program is an ordinary device function that the
// block trampoline (pto::b200::launch / PTO_B200_LAUNCH) runs on every thread block, so after this header
// `__global__` expands to nothing.  Code that needs CUDA's own kernel attribute afterwards can use
// PTO_B200_CUDA_GLOBAL, or define PTO_B200_KEEP_CUDA_GLOBAL before including this header.
#pragma once

#if !defined(__CUDACC__)
#error "the B200 backend of the PTO ISA is compiled with nvcc (sm_100a)"
#endif

#include "b200/types.hpp"
#include "b200/tile.hpp"
#include "b200/runtime.hpp"
#include "b200/event.hpp"
#include "b200/instr.hpp"
#include "b200/pipe.hpp"

#define PTO_B200_CUDA_GLOBAL __attribute__((global))

#if !defined(PTO_B200_KEEP_CUDA_GLOBAL)
#undef __global__
#define __global__
#endif
