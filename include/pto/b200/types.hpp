// PTO type surface for the B200 (sm_100a) backend: qualifier macros, enums, pipes and events.
// Names and enumerator values follow the PTO ISA headers of the reference
// (include/pto/common/type.hpp:92-252, include/pto/common/memory.hpp:19-43, include/pto/common/event.hpp:14,
// include/pto/common/cpu_stub.hpp:29-53; paths relative to the reference root) so that tile programs written
// against them compile here.  On this backend one CUDA thread block plays the role of one AI core.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

// ---------------------------------------------------------------- qualifiers
// Tile programs mark every function AICORE.  Here such a function is compiled for both sides: the device
// side does the work, the host side is an empty shell so that host code which names a kernel (as the
// reference's CPU-simulation launchers do) still compiles.
#define AICORE __host__ __device__
#define PTO_INLINE __forceinline__
#define PTO_INST __host__ __device__ __forceinline__
#define PTO_INTERNAL __host__ __device__ __forceinline__
// bodies that are kept out of line so that a tile program's instruction stream stays small (one copy per instance)
#define PTO_B200_OUTLINE __device__ __noinline__
#define __aicore__
#define __gm__
#define __ubuf__
#define __cbuf__
#define __ca__
#define __cb__
#define __cc__
#define __fbuf__
#define __in__
#define __out__
#define __tf__

#if defined(__CUDA_ARCH__)
#define PTO_B200_DEVICE_CODE 1
#else
#define PTO_B200_DEVICE_CODE 0
#endif

using half = __half;
using aclFloat16 = __half;
using bfloat16_t = __nv_bfloat16;
// operand and scale types of the MX block-scaled product (include/pto/common/type.hpp in the reference)
using float8_e4m3_t = __nv_fp8_e4m3;
using float8_e5m2_t = __nv_fp8_e5m2;
using float8_e8m0_t = __nv_fp8_e8m0;
typedef void *aclrtStream;

// ---------------------------------------------------------------- pipes and events
enum pipe_t : int {
    PIPE_S = 0,
    PIPE_V = 1,
    PIPE_MTE1 = 2,
    PIPE_MTE2 = 3,
    PIPE_MTE3 = 4,
    PIPE_M = 5,
    PIPE_ALL = 6,
    PIPE_FIX = 7,
};

enum event_t : int {
    EVENT_ID0 = 0,
    EVENT_ID1,
    EVENT_ID2,
    EVENT_ID3,
    EVENT_ID4,
    EVENT_ID5,
    EVENT_ID6,
    EVENT_ID7,
};
constexpr int EVENT_ID_MAX = 8;

namespace pto {

constexpr int DYNAMIC = -1;

enum class TileType { Vec, Mat, Left, Right, Acc, Bias, Scaling, ScaleLeft, ScaleRight };
enum class BLayout { RowMajor = 0, ColMajor = 1 };
enum class SLayout { NoneBox = 0, RowMajor = 1, ColMajor = 2 };

enum class Layout { ND, DN, NZ };

enum class MaskPattern : uint8_t { P0101 = 1, P1010 = 2, P0001 = 3, P0010 = 4, P0100 = 5, P1000 = 6, P1111 = 7 };

enum class RoundMode : uint8_t {
    CAST_NONE = 0,
    CAST_RINT = 1,  // to nearest, ties to even
    CAST_ROUND = 2, // to nearest, ties away from zero
    CAST_FLOOR = 3,
    CAST_CEIL = 4,
    CAST_TRUNC = 5,
    CAST_ODD = 6,
};

enum class PadValue { Null, Zero, Max, Min };
// include/pto/common/type.hpp:131-139
enum class CmpMode : uint8_t { EQ = 0, NE = 1, LT = 2, LE = 3, GT = 4, GE = 5 };
enum class CompactMode { Null, Normal };
enum class SaturationMode : uint8_t { ON = 0, OFF = 1 };
enum class AtomicType : uint8_t { AtomicNone = 0, AtomicAdd = 1 };
enum class AccPhase : uint8_t { Unspecified = 0x0, Unknown = Unspecified, Partial = 0x2, Final = 0x3 };
enum class STPhase : uint8_t { Unspecified = 0x0, Partial = 0x2, Final = 0x3 };
enum class ReluPreMode : uint8_t { NoRelu = 0, NormalRelu = 1 };

namespace GlobalTensorDim {
constexpr int DIM_0 = 0;
constexpr int DIM_1 = 1;
constexpr int DIM_2 = 2;
constexpr int DIM_3 = 3;
constexpr int DIM_4 = 4;
constexpr int TOTAL_DIM = 5;
} // namespace GlobalTensorDim

struct TileConfig {
    static constexpr int alignedSize = 32;    // bytes
    static constexpr int fixedRowSize = 16;
    static constexpr int fixedColSize = 16;
    static constexpr int fixedMxRowSize = 16;
    static constexpr int fixedMxColSize = 2;
    static constexpr int fractalABSize = 512;
    static constexpr int fractalCSize = 1024;
    static constexpr int fractalMxSize = 32;
};

// What an instruction returns; assigning it to an Event raises that event's flag (event.hpp).
struct RecordEvent {};

// geometry constants of the ISA that tile programs refer to
constexpr int BLOCK_BYTE_SIZE = 32;
constexpr int C0_SIZE_BYTE = 32;
constexpr int FRACTAL_NZ_ROW = 16;
constexpr int BLOCK_LEN = 16;
constexpr int CUBE_BLOCK_SIZE = 512;

} // namespace pto
