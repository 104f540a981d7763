// Per-block execution context of the PTO backend for B200, and the host-side launch helper.
//
// One thread block (256 threads) is one "AI core".  All threads run the same instruction stream of the
// tile program; every PTO instruction is executed cooperatively by the block.  Dynamic shared memory holds
//   [ control | arena ]
// control = the tensor-memory base, the table of flags (one mbarrier per (source pipe, destination pipe,
// event id), the direct counterpart of the reference's set_flag / wait_flag, include/pto/common/cpu_stub.hpp:
// 85-86 and docs/coding/Event.md in the reference) and each warp's flag phases; arena = the space that TASSIGN
// addresses index into.  The NPU has separate address spaces for L1 / UB (Mat and Vec tiles), L0A (Left) and
// L0B (Right), each starting at 0; here they are windows of the one arena:
//   Vec, Mat : [0, PTO_B200_L0A_OFFSET)            default 96 KiB  (two 128x64 + two 64x256 fp16 staging tiles)
//   Left     : [PTO_B200_L0A_OFFSET, PTO_B200_L0B_OFFSET)   48 KiB  (ping at 0, pong at 32 KiB, 16 KiB each)
//   Right    : [PTO_B200_L0B_OFFSET, end of arena)          64 KiB+ (ping at 0, pong at 32 KiB, 32 KiB each)
//   Bias     : a 1 KiB table in the control block (one row of up to 256 floats for TMATMUL_BIAS)
//   ScaleLeft / ScaleRight : the last two 4 KiB of the arena (scale atoms of TMATMUL_MX)
// Define the two macros before including the PTO headers to move the windows for a whole translation unit, or give
// the offsets per launch (LaunchOptions).
// 512 tensor-memory columns are allocated per block for Acc tiles.
//
// Every wait of a tile program (wait_flag, wait_flag_dev, Event::Wait) is bounded: the launch carries a limit in
// nanoseconds (two seconds unless the caller gives one); a wait that runs out records the flag it waited for,
// raises the block's abort flag so that all later waits return at once, and the block epilogue writes
// {code 4, block, flag index, source / destination pipes} into the caller's status record.  Nothing traps.
#pragma once

#include <cuda.h>

#include "tile.hpp"

namespace pto {
namespace b200 {

#ifndef PTO_B200_L0A_OFFSET
#define PTO_B200_L0A_OFFSET (96 * 1024)
#endif
#ifndef PTO_B200_L0B_OFFSET
#define PTO_B200_L0B_OFFSET (144 * 1024)
#endif

constexpr int kBlockThreads = 256;
constexpr int kNumPipes = 8;
constexpr int kNumFlags = kNumPipes * kNumPipes * EVENT_ID_MAX; // 512
constexpr int kTmemCols = 512;
constexpr unsigned long long kWaitLimitNs = 2000000000ull; // default limit of a wait
constexpr int kNumDevFlags = 16;   // cross-core flag ids (wait_flag_dev / ffts_cross_core_sync)
constexpr int kNumCoreStatics = 2; // function-local statics of tile programs (see PTO_B200_CORE_STATIC)
constexpr int kWarps = kBlockThreads / 32;
// How a launch runs its program (LaunchOptions):
//   kModeInOrder   every instruction completes before the next one starts
//   kModePipeWarps the pipes of the core run on warps of their own (teams, below); every warp walks the whole
//                  instruction stream and skips what is not its own, and flags are raised and awaited by the warps of
//                  the pipes they name
//   kModeViews     TEXTRACT / TMOV of an aligned window hands the operand tile a view of the staged tile (no copy)
//   kModeEngineLoads every TLOAD is a copy by the copy engine, prepared ahead of time by a thread of its own
constexpr int kModeInOrder = 1, kModePipeWarps = 2, kModeViews = 4, kModeEngineLoads = 8;
constexpr int kModeTmemColsShift = 8; // bits 8..17: the tensor-memory columns the block allocates (LaunchOptions::tmem_cols)
// kModePipeWarps is a property of the translation unit: define PTO_B200_PIPE_WARPS before including the PTO header and
// every tile program of the unit runs with its pipes on warps of their own (LaunchOptions::pipe_warps must say the
// same).  The instructions then know at compile time which threads execute them.
#ifdef PTO_B200_PIPE_WARPS
constexpr bool kPipeWarps = true;
#else
constexpr bool kPipeWarps = false;
#endif
constexpr int kTeamLThreads = 32;   // warp 1: the threads that copy tiles for MTE2 where the copy engine does not
constexpr int kTmemWarp = 2;        // the warp without a pipe allocates and frees the block's tensor memory
constexpr int kTeamBWarp = 3;
constexpr int kTeamCFirstWarp = 4, kTeamCThreads = 128; // warps 4..7
// TSTORE's staging area (LaunchOptions::store_staging_offset)
constexpr uint32_t kStoreStagingRowBytes = 128 + 16; // a 128-byte row piece per thread, padded against bank conflicts
constexpr uint32_t kStoreStagingBytes = 128 * kStoreStagingRowBytes;
constexpr uint32_t kNoStoreStaging = 0xffffffffu;
constexpr int kNotAMember = 1 << 20; // thread index handed to threads outside the executing team: their loops are empty

// What a block reports when one of its waits ran out (same layout as the status record of libpto_b200.so).
struct StatusRecord {
    int code;   // 0 ok, 4 = a wait gave up
    int block;  // block index that reported
    int where;  // index of the flag waited for: ((src pipe * 8 + dst pipe) * 8 + event id); 512 + id for a cross-core flag;
                // 600 + n: an instruction that pipe_warps does not cover; 601: a TLOAD that the copy engine cannot do in
                // a launch with engine_loads; 602: a tile assigned beyond the arena; 1024 + flag: a raise that waited for
                // the previous one to be consumed; 1536 / 1537: the loading / preparing thread waiting for the other
    int detail; // src pipe * 16 + dst pipe
};

struct Control {
    uint32_t tmem_base;
    int abort_flag;
    int mode;                       // kModeInOrder | kModePipeWarps | kModeViews (LaunchOptions)
    int fail_where;                 // flag index of the first wait that gave up
    unsigned long long wait_limit_ns;
    uint64_t flags[kNumFlags];
    uint32_t phase[kNumFlags / 32][kWarps];              // phase bit of every flag, per warp
    uint8_t bias_table[1024];                            // the address space of TileType::Bias tiles (the NPU's bias table)
    int dev_flags[kNumDevFlags];                         // counting flags between the cube and vector roles of a core
    uint32_t event_next[kWarps][kNumPipes * kNumPipes / 8]; // next automatic event id of a pipe pair (4 bits each), per warp
    unsigned long long core_static[kNumCoreStatics][kWarps]; // function-local statics of tile programs, per warp
    uint32_t core_static_init[kWarps];                   // bit s set: slot s of this warp holds a value
    uint32_t l0a_offset;                                 // start of the Left window of the arena (bytes)
    uint32_t l0b_offset;                                 // start of the Right window of the arena (bytes)
    // pipe_warps: how often each flag was raised and how many of its waits are complete (modulo 256).  A flag is an
    // mbarrier, which tells "this phase" from "the one before" and no further; a team that runs ahead of the flag's
    // waiters raises it again only once the previous raise has been consumed (see set_flag).
    uint8_t raised[kNumFlags];
    uint8_t consumed[kNumFlags];
};
constexpr int kControlBytes = ((int)sizeof(Control) + 1023) / 1024 * 1024;
static_assert(kControlBytes == 7 * 1024, "the control block is 7 KiB: the arena is the other 220 KiB");
constexpr int kDefaultSmemBytes = 227 * 1024; // control (7 KiB) + 220 KiB arena; the buffer is declared 1 KiB aligned
constexpr uint32_t kArenaBytes = kDefaultSmemBytes - kControlBytes;
// scale tiles of the MX product (TileType::ScaleLeft / ScaleRight) have windows of their own at the end of the arena:
// 4 KiB each (a program that uses them keeps its Right window below 212 KiB)
constexpr uint32_t kScaleRightOffset = 212 * 1024;
constexpr uint32_t kScaleLeftOffset = 216 * 1024;
// tensor-memory columns kept for the scales of TMATMUL_MX (accumulators of such a program stay below them)
constexpr uint32_t kMxScaleTmemCol = 480;

#ifdef PTO_B200_TIMELINE
// Profiling aid, compiled in with -DPTO_B200_TIMELINE: the first thread of each team of block 0 (of the whole block
// without pipe_warps: thread 0) stamps (code, clock64) at the entry and exit of flags and instructions.
// Codes: 0x1000 + flag / 0x2000 + flag: wait_flag entered / passed; 0x3000 + flag / 0x3800 + flag: set_flag entered /
// done; 0x4000 / 0x4001 TLOAD; 0x5000 / 0x5001 TEXTRACT; 0x6000 / 0x6001 TMATMUL; 0x7000 / 0x7001 TSTORE.
constexpr int kTimelineEntries = 4096;
static __device__ unsigned long long g_timeline[3][kTimelineEntries];
static __device__ unsigned int g_timeline_n[3];
#endif
// Matrices in global memory that a launch registers so that TLOAD can fetch tiles of them with the copy engine (TMA):
// a tile program builds its GlobalTensors from raw pointers on the device, where a tensor map cannot be encoded, so the
// launch encodes one map per registered matrix (rows of `pitch` elements, a box of 128 bytes x `box_rows` rows, 128-byte
// swizzle) and TLOAD turns a tile's address into coordinates of the matrix it lies in.  Tiles of unregistered memory are
// fetched with cp.async.  Used with pipe_warps.
constexpr int kMaxTmaRegions = 4;
struct TmaRegion {
    const void *base = nullptr; // element (0, 0) of a row-major matrix, 16-byte aligned
    uint64_t rows = 0, cols = 0; // extent in elements
    uint64_t pitch = 0;          // elements between rows (pitch * elem_bytes a multiple of 16)
    int elem_bytes = 2;
    uint32_t box_rows = 128;     // rows one copy moves (a power of two, at most 256); a tile's lines are a multiple of it
};
struct TmaTable {
    CUtensorMap map[kMaxTmaRegions];
    unsigned long long base[kMaxTmaRegions];
    unsigned long long bytes[kMaxTmaRegions];       // base .. base + bytes holds the matrix
    unsigned long long pitch_bytes[kMaxTmaRegions];
    unsigned long long row_bytes[kMaxTmaRegions];   // cols * elem_bytes
    uint32_t box_rows[kMaxTmaRegions];
    uint32_t elem_bytes[kMaxTmaRegions];
    int count;
};

#if PTO_B200_DEVICE_CODE
// The block's dynamic shared memory, declared 1 KiB aligned (the swizzled operand layouts want that).  The launch
// trampoline checks the address and reports instead of running the program if the declaration was not honoured.
__device__ __forceinline__ uint8_t *smem_base()
{
    extern __shared__ __align__(1024) uint8_t pto_b200_dynamic_smem[];
    return pto_b200_dynamic_smem;
}
__device__ __forceinline__ Control *control()
{
    return reinterpret_cast<Control *>(smem_base());
}
__device__ __forceinline__ uint8_t *arena()
{
    return smem_base() + kControlBytes;
}
// start of the window of the arena that tiles of a location index into
template <TileType Loc>
__device__ __forceinline__ uint8_t *arena_of()
{
    if constexpr (Loc == TileType::Bias) {
        return control()->bias_table;
    } else {
        if constexpr (Loc == TileType::Left) {
            return arena() + control()->l0a_offset;
        } else if constexpr (Loc == TileType::Right) {
            return arena() + control()->l0b_offset;
        } else if constexpr (Loc == TileType::ScaleLeft) {
            return arena() + kScaleLeftOffset;
        } else if constexpr (Loc == TileType::ScaleRight) {
            return arena() + kScaleRightOffset;
        } else {
            return arena();
        }
    }
}
// Does a tile of `bytes` at offset `addr` of the window of `Loc` lie inside the arena?  Instructions that write whole
// matrix tiles check this and report {4, block, 602} instead of writing past the block's shared memory (a tile
// assigned beyond its window's room is a program error that would otherwise fault the GPU).
// the arena of this launch: its dynamic shared memory less the control block (LaunchOptions::smem_bytes)
__device__ __forceinline__ uint32_t arena_bytes()
{
    uint32_t total;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(total));
    return total - static_cast<uint32_t>(kControlBytes);
}
template <TileType Loc>
__device__ __forceinline__ bool tile_in_arena(uint32_t addr, uint32_t bytes)
{
    const uint32_t start = static_cast<uint32_t>(arena_of<Loc>() - arena()) + addr;
    const uint32_t room = arena_bytes();
    return start <= room && bytes <= room - start;
}
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ int flag_index(int src, int dst, int id)
{
    return ((src & 7) * kNumPipes + (dst & 7)) * EVENT_ID_MAX + (id & 7);
}

// The bump allocator behind freshly constructed tiles (tile.hpp).  A pipe has no flags with itself (pipe_barrier
// orders a pipe with itself), so the eight flag words of PIPE_S -> PIPE_S are never barriers: they hold the
// allocator's counters, four 16-bit counters per warp (every lane of a warp constructs the same tiles in the same
// order, and so does every warp of a block, so all threads arrive at the same addresses without exchanging any).
// Counters are in units of 1 KiB for the shared-memory windows (the swizzled layouts want that alignment) and of
// 32 columns for tensor memory.
static_assert(PIPE_S == 0 && kWarps * 4 * sizeof(uint16_t) == EVENT_ID_MAX * sizeof(uint64_t),
              "the tile allocator's counters occupy the flag words of PIPE_S -> PIPE_S");
__device__ __forceinline__ uint32_t tile_auto_place(int space, uint32_t amount)
{
    Control *c = control();
    volatile uint16_t *ctr = reinterpret_cast<volatile uint16_t *>(&c->flags[0]) + (threadIdx.x >> 5) * 4 + space;
    const bool tmem = space == kSpaceAcc;
    const uint32_t unit = tmem ? 32u : 1024u;
    const uint32_t want = (amount + unit - 1) / unit;
    uint32_t limit;
    if (tmem) {
        limit = kTmemCols / 32;
    } else if (space == kSpaceVec) {
        limit = (c->l0a_offset < c->l0b_offset ? c->l0a_offset : c->l0b_offset) / 1024u;
    } else if (space == kSpaceLeft) {
        limit = ((c->l0b_offset > c->l0a_offset ? c->l0b_offset : kScaleRightOffset) - c->l0a_offset) / 1024u;
    } else {
        limit = ((c->l0a_offset > c->l0b_offset ? c->l0a_offset : kScaleRightOffset) - c->l0b_offset) / 1024u;
    }
    __syncwarp();
    const uint32_t at = *ctr;
    __syncwarp();
    if (at + want > limit) {
        return 0; // the window is used up: the tile has to be assigned an address before it is used
    }
    if ((threadIdx.x & 31) == 0) {
        *ctr = static_cast<uint16_t>(at + want);
    }
    __syncwarp();
    return at * unit;
}

// ---- teams: who executes an instruction.  Without PTO_B200_PIPE_WARPS the whole block does.  With it:
//   MTE2          thread 0 raises and awaits the pipe's flags and hands tiles of registered matrices to the copy
//                 engine; warp 1 (team L) copies where a tile is copied by threads (cp.async, vector tiles)
//   MTE1 and M    the first thread of warp 3 (team B): operand windows and the products, issued by one thread
//   V, MTE3, FIX, S   warps 4..7 (team C): vector work and stores; four warps, so that together they reach every
//                 tensor-memory lane
// Warp 2 has no pipe; the other lanes of warps 0 and 3 leave when the block begins (a thread that works alone is not
// held up by lanes of its warp that wait at barriers).  Every warp walks the whole instruction stream; an instruction does its work on the threads of
// its pipe and nothing on the others (their thread index is kNotAMember, which empties every loop).
__device__ __forceinline__ constexpr bool pipe_warps()
{
    return kPipeWarps;
}
enum : int { kTeamL = 0, kTeamB = 1, kTeamC = 2 };
__device__ __forceinline__ int team_of_pipe(int pipe)
{
    return pipe == PIPE_MTE2 ? kTeamL : ((pipe == PIPE_MTE1 || pipe == PIPE_M) ? kTeamB : kTeamC);
}
__device__ __forceinline__ int team_threads(int team)
{
    return team == kTeamL ? kTeamLThreads : (team == kTeamB ? 1 : kTeamCThreads);
}
__device__ __forceinline__ int team_first_thread(int team)
{
    return team == kTeamL ? 32 : (team == kTeamB ? kTeamBWarp * 32 : kTeamCFirstWarp * 32);
}
template <int kTeam>
__device__ __forceinline__ int team_tid()
{
    if (!pipe_warps()) {
        return threadIdx.x;
    }
    const int t = static_cast<int>(threadIdx.x) - team_first_thread(kTeam);
    return (t >= 0 && t < team_threads(kTeam)) ? t : kNotAMember;
}
template <int kTeam>
__device__ __forceinline__ int team_size()
{
    return pipe_warps() ? team_threads(kTeam) : static_cast<int>(blockDim.x);
}
template <int kTeam>
__device__ __forceinline__ void team_sync()
{
    if (!pipe_warps()) {
        __syncthreads();
    } else if (kTeam == kTeamL) {
        // the loading thread (alone in warp 0) and the copying warp
        if (threadIdx.x == 0 || (threadIdx.x >> 5) == 1) {
            asm volatile("bar.sync 1, 64;" ::: "memory");
        }
    } else if (kTeam == kTeamC && team_tid<kTeam>() != kNotAMember) {
        asm volatile("bar.sync 3, %0;" ::"n"(kTeamCThreads) : "memory");
    }
}
// does this thread raise and await the flags of `pipe` (and execute its instructions)?
__device__ __forceinline__ bool runs(int pipe)
{
    if (!pipe_warps()) {
        return true;
    }
    const int team = team_of_pipe(pipe);
    if (team == kTeamL) {
        return threadIdx.x == 0;
    }
    const int t = static_cast<int>(threadIdx.x) - team_first_thread(team);
    return t >= 0 && t < team_threads(team);
}
// the threads that copy tiles for MTE2 where the copy engine does not
__device__ __forceinline__ bool helps_mte2()
{
    return !pipe_warps() || threadIdx.x == 0 || (threadIdx.x >> 5) == 1;
}
// vector, store and scalar instructions (team C) are the default
__device__ __forceinline__ int tid() { return team_tid<kTeamC>(); }
__device__ __forceinline__ int nthreads() { return team_size<kTeamC>(); }
__device__ __forceinline__ void sync() { team_sync<kTeamC>(); }
__device__ __forceinline__ int tid_l() { return team_tid<kTeamL>(); }
__device__ __forceinline__ int nthreads_l() { return team_size<kTeamL>(); }
__device__ __forceinline__ void sync_l() { team_sync<kTeamL>(); }
__device__ __forceinline__ int tid_b() { return team_tid<kTeamB>(); }
__device__ __forceinline__ int nthreads_b() { return team_size<kTeamB>(); }
__device__ __forceinline__ void sync_b() { team_sync<kTeamB>(); }
// An instruction that pipe_warps does not cover (its work needs threads of two teams): reported through the status
// record (where = 600 + what) and skipped; the program's waits return at once from then on.
__device__ __forceinline__ bool not_with_pipe_warps(int what)
{
    if (!pipe_warps()) {
        return false;
    }
    Control *c = control();
    if ((threadIdx.x & 31) == 0 && c->abort_flag == 0) {
        c->fail_where = 600 + what;
        c->abort_flag = 1;
    }
    return true;
}
__device__ __forceinline__ void stamp(int code)
{
#ifdef PTO_B200_TIMELINE
    if (blockIdx.x != 0) {
        return;
    }
    int team = -1;
    if (!pipe_warps()) {
        team = threadIdx.x == 0 ? 0 : -1;
    } else if (threadIdx.x == 0) {
        team = kTeamL;
    } else if (threadIdx.x == kTeamBWarp * 32) {
        team = kTeamB;
    } else if (threadIdx.x == kTeamCFirstWarp * 32) {
        team = kTeamC;
    }
    if (team >= 0) {
        // the running count lives in shared memory (the unused flag words of PIPE_MTE1 -> PIPE_MTE1): a stamp costs one
        // shared-memory round trip and two stores
        volatile uint32_t *count = reinterpret_cast<volatile uint32_t *>(&control()->flags[flag_index(PIPE_MTE1, PIPE_MTE1, 0)]) + team;
        const unsigned int i = *count;
        if (i < kTimelineEntries) {
            g_timeline[team][i] = (static_cast<unsigned long long>(code) << 48) | (clock64() & 0xffffffffffffull);
            *count = i + 1;
            g_timeline_n[team] = i + 1;
        }
    }
#else
    (void)code;
#endif
}
// Views handed out by TEXTRACT (kModeViews) keep the staged tile in use until the products that read them are
// complete.  A set_flag(PIPE_MTE1, PIPE_MTE2, id) that follows such a TEXTRACT ("the staged tile may be loaded
// again") is therefore held back and raised by the tensor core itself (tcgen05.commit) at the next flag that the
// matrix pipe raises, which in program order comes after the products that read the views.  The list of flags held
// back lives in the flag words of PIPE_V -> PIPE_V (a pipe has no flags with itself); only the thread that issues the
// products touches it.
__device__ __forceinline__ uint32_t *held_back()
{
    return reinterpret_cast<uint32_t *>(&control()->flags[flag_index(PIPE_V, PIPE_V, 0)]);
}
constexpr int kMaxHeldBack = 12;
// held_back()[14]: tiles were written through the generic proxy (cp.async loads, copying TEXTRACT / TMOV) since the
// block began: waits then order those writes before the tensor core's reads with a proxy fence

// The launch's table of registered matrices (a kernel parameter; its address is kept in the flag words of
// PIPE_MTE2 -> PIPE_MTE2) and the loads that TLOAD has prepared but not yet issued (flag words of PIPE_MTE3 -> PIPE_MTE3):
// a copy by the copy engine completes on an mbarrier named when it is issued, and the flag that a load raises is only
// known at the set_flag that follows it, so TLOAD records the copy and set_flag(PIPE_MTE2, ...) issues it.
struct PendingLoad {   // everything the copy instructions need, ready to use
    unsigned long long map; // address of the matrix's tensor map
    uint32_t dst;           // shared-memory address of the tile
    uint32_t x, y;          // element coordinates of the tile's first element
    uint32_t shape;         // bits 0..7 128-byte blocks along the contiguous dimension, 8..15 boxes along the lines,
                            // 16..23 log2 of the box's rows, 24..31 elements per 128-byte block
};
constexpr int kMaxPendingLoads = 2;
__device__ __forceinline__ const TmaTable *&tma_table()
{
    return *reinterpret_cast<const TmaTable **>(&control()->flags[flag_index(PIPE_MTE2, PIPE_MTE2, 0)]);
}
__device__ __forceinline__ volatile uint32_t *pending_count()
{
    return reinterpret_cast<volatile uint32_t *>(&control()->flags[flag_index(PIPE_MTE3, PIPE_MTE3, 0)]);
}
__device__ __forceinline__ PendingLoad *pending_loads()
{
    return reinterpret_cast<PendingLoad *>(reinterpret_cast<uint8_t *>(&control()->flags[flag_index(PIPE_MTE3, PIPE_MTE3, 0)]) + 16);
}
static_assert(16 + kMaxPendingLoads * sizeof(PendingLoad) <= 64, "pending loads fit the eight flag words");
// what TLOAD needs of the registered matrices, copied from the kernel parameter into shared memory when the block
// begins (flag words of PIPE_M -> PIPE_M and PIPE_ALL -> PIPE_ALL)
struct RegionBounds { // 64 bytes
    unsigned long long base[kMaxTmaRegions];
    unsigned long long end[kMaxTmaRegions];
};
struct RegionShapes { // 52 bytes
    uint32_t pitch_bytes[kMaxTmaRegions];
    uint32_t row_bytes[kMaxTmaRegions];
    uint16_t box_rows[kMaxTmaRegions];
    uint8_t elem_bytes[kMaxTmaRegions];
    uint32_t count;
};
__device__ __forceinline__ uint32_t log2_pow2(uint32_t v)
{
    return 31u - static_cast<uint32_t>(__clz(static_cast<int>(v)));
}
static_assert(sizeof(RegionBounds) <= 64 && sizeof(RegionShapes) <= 64, "region caches fit eight flag words each");
__device__ __forceinline__ RegionBounds *region_bounds()
{
    return reinterpret_cast<RegionBounds *>(&control()->flags[flag_index(PIPE_M, PIPE_M, 0)]);
}
__device__ __forceinline__ RegionShapes *region_shapes()
{
    return reinterpret_cast<RegionShapes *>(&control()->flags[flag_index(PIPE_ALL, PIPE_ALL, 0)]);
}
// floor(2^32 / pitch) per registered matrix (flag words of PIPE_FIX -> PIPE_FIX): a row number is then a multiply-high
// and at most two corrections instead of an integer division
__device__ __forceinline__ uint32_t *region_reciprocals()
{
    return reinterpret_cast<uint32_t *>(&control()->flags[flag_index(PIPE_FIX, PIPE_FIX, 0)]);
}
// LaunchOptions::engine_loads: the copies that TLOADs become are prepared (matrix found, coordinates computed) by the
// first thread of warp 1, which walks the instruction stream ahead of the loading thread: no flag holds it, only this
// ring of two prepared copies (flag words of PIPE_FIX -> PIPE_FIX, behind the reciprocals).  The loading thread counts
// the TLOADs it passes (`taken`) and issues the prepared copies at the set_flag that follows (`issued`); the preparing
// thread fills entry `head` when head - issued < 2.  Counters live beside the table's address (PIPE_MTE2 -> PIPE_MTE2).
constexpr uint32_t kLoadRing = 2;
constexpr int kPrepareThread = 32;
__device__ __forceinline__ PendingLoad *load_ring()
{
    return reinterpret_cast<PendingLoad *>(reinterpret_cast<uint8_t *>(&control()->flags[flag_index(PIPE_FIX, PIPE_FIX, 0)]) + 16);
}
__device__ __forceinline__ volatile uint32_t *load_ring_counters() // [0] head, [1] taken, [2] issued
{
    return reinterpret_cast<volatile uint32_t *>(reinterpret_cast<uint8_t *>(&control()->flags[flag_index(PIPE_MTE2, PIPE_MTE2, 0)]) + 8);
}
__device__ __forceinline__ uint32_t divide_by_pitch(uint32_t o, uint32_t pitch, uint32_t reciprocal, uint32_t &remainder)
{
    uint32_t q = __umulhi(o, reciprocal); // never above the quotient, below it by at most two
    uint32_t r = o - q * pitch;
    if (r >= pitch) {
        q += 1, r -= pitch;
    }
    if (r >= pitch) {
        q += 1, r -= pitch;
    }
    remainder = r;
    return q;
}
// [1] of the pending block: TLOAD's decision for the team (1: the copy engine fetches the tile, 0: cp.async)
 // held_back()[13]: 1 + arena offset of TSTORE's staging area, 0 = none

// ---- mbarrier primitives (bounded waits: a wait that runs out raises the block's abort flag)
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// arrives once all cp.async copies issued so far by this thread have landed
__device__ __forceinline__ void mbar_arrive_after_copies(uint64_t *bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    return now;
}
// the first wait of a block that gives up records what it waited for; every later wait returns at once
__device__ __forceinline__ void give_up(int where)
{
    Control *ctl = control();
    if (atomicCAS(&ctl->abort_flag, 0, 1) == 0) {
        ctl->fail_where = where;
    }
}
// waits (bounded like every wait) until *word - base >= least, counters taken modulo 2^32
__device__ __noinline__ bool wait_for_count(volatile uint32_t *word, uint32_t least, int where)
{
    Control *ctl = control();
    volatile int *abort_flag = &ctl->abort_flag;
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (static_cast<int32_t>(*word - least) >= 0) {
            return true;
        }
        if ((i & 0x3f) == 0x3f) {
            if (*abort_flag) {
                return false;
            }
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > ctl->wait_limit_ns) {
                break;
            }
        }
    }
    give_up(where);
    return false;
}

__device__ __noinline__ bool mbar_wait_slow(uint64_t *bar, uint32_t parity, int where)
{
    Control *ctl = control();
    volatile int *abort_flag = &ctl->abort_flag;
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((i & 0x3f) == 0x3f) {
            if (*abort_flag) {
#ifdef PTO_B200_TRACE_WAITS
                // debugging aid: which wait each warp of block 0 was held in when the block gave up
                if (t0 != 0 && blockIdx.x == 0 && (threadIdx.x & 31) == 0) {
                    printf("pto wait trace: warp %d held in flag %d (src %d dst %d id %d) parity %u\n", threadIdx.x >> 5, where,
                           (where >> 6) & 7, (where >> 3) & 7, where & 7, parity);
                }
#endif
                return false;
            }
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > ctl->wait_limit_ns) {
                break; // the launch's limit on the global timer: give up instead of hanging the device
            }
            if (i > 4096) {
                __nanosleep(64);
            }
        }
    }
#ifdef PTO_B200_TRACE_WAITS
    if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) {
        printf("pto wait trace: warp %d gave up on flag %d (src %d dst %d id %d) parity %u\n", threadIdx.x >> 5, where,
               (where >> 6) & 7, (where >> 3) & 7, where & 7, parity);
    }
#endif
    give_up(where);
    return false;
}

// the first poll inline, the bounded polling loop out of line (a tile program has dozens of waits)
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int where = -1)
{
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    return mbar_wait_slow(bar, parity, where);
}

// pipe_warps: before flag `f` is raised for the n-th time, its first n - 1 raises must have been consumed (bounded
// like every wait; see Control::raised)
__device__ __noinline__ bool wait_until_consumed_slow(int f, uint8_t n)
{
    Control *ctl = control();
    volatile uint8_t *consumed = &ctl->consumed[f];
    volatile int *abort_flag = &ctl->abort_flag;
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (*consumed == n) {
            return true;
        }
        if ((i & 0x3f) == 0x3f) {
            if (*abort_flag) {
                return false;
            }
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > ctl->wait_limit_ns) {
                break;
            }
        }
    }
#ifdef PTO_B200_TRACE_WAITS
    if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) {
        printf("pto wait trace: warp %d gave up raising flag %d for the %u-th time (consumed %u)\n", threadIdx.x >> 5, f, n, *consumed);
    }
#endif
    give_up(1024 + f);
    return false;
}

__device__ __forceinline__ bool wait_until_consumed(int f, uint8_t n)
{
    if (*reinterpret_cast<volatile uint8_t *>(&control()->consumed[f]) == n) {
        return true;
    }
    return wait_until_consumed_slow(f, n);
}

// ---- loads by the copy engine
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint64_t *bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// issues the loads that TLOAD prepared, completing on `bar` (called by the first thread of team L before it arrives)
// the copy instructions of up to two prepared copies, completing on `bar` (entries already in registers: each copy
// instruction is a compiler barrier for memory)
__device__ __forceinline__ void issue_copies(uint64_t *bar, const PendingLoad (&e)[2], uint32_t n)
{
    uint32_t bytes = 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (static_cast<uint32_t>(i) < n) {
            bytes += ((e[i].shape & 0xffu) * ((e[i].shape >> 8) & 0xffu)) << (((e[i].shape >> 16) & 0xffu) + 7u);
        }
    }
    mbar_expect_tx(bar, bytes);
    const uint32_t bar_s = smem_u32(bar);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (static_cast<uint32_t>(i) < n) {
            const uint32_t blocks = e[i].shape & 0xffu, boxes = (e[i].shape >> 8) & 0xffu, log2_rows = (e[i].shape >> 16) & 0xffu;
            const int block_elems = static_cast<int>(e[i].shape >> 24);
            const uint32_t box_bytes = 128u << log2_rows, pitch = boxes * box_bytes;
            for (uint32_t b = 0; b < blocks; ++b) {
                for (uint32_t l = 0; l < boxes; ++l) {
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                            e[i].dst + b * pitch + l * box_bytes),
                        "l"(e[i].map), "r"(bar_s), "r"(static_cast<int>(e[i].x) + static_cast<int>(b) * block_elems),
                        "r"(static_cast<int>(e[i].y + (l << log2_rows))));
                }
            }
        }
    }
}
static_assert(kMaxPendingLoads == 2 && kLoadRing == 2, "issue_copies takes two entries");

// issues the loads that TLOAD prepared, completing on `bar` (called by the loading thread before it arrives)
__device__ __noinline__ void issue_pending_loads(uint64_t *bar)
{
    PendingLoad e[2];
    if (control()->mode & kModeEngineLoads) {
        volatile uint32_t *c = load_ring_counters();
        const uint32_t taken = c[1], issued = c[2];
        const uint32_t n = taken - issued;
        if (n == 0) {
            return;
        }
        if (!wait_for_count(&c[0], taken, 1536)) { // the preparing thread has filled the entries
            return;
        }
        const PendingLoad *ring = load_ring();
        bool ok = true;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (static_cast<uint32_t>(i) < n) {
                const PendingLoad *p = ring + ((issued + i) & (kLoadRing - 1));
                e[i].map = p->map, e[i].dst = p->dst, e[i].x = p->x, e[i].y = p->y, e[i].shape = p->shape;
                ok = ok && e[i].shape != 0;
            }
        }
        if (!ok) {
            give_up(601); // a TLOAD that the copy engine cannot do, in a launch that promised there are none
            c[2] = taken;
            return;
        }
        issue_copies(bar, e, n);
        c[2] = taken; // the entries may be filled again
        return;
    }
    volatile uint32_t *count = pending_count();
    const uint32_t n = *count;
    if (n == 0) {
        return;
    }
    const PendingLoad *p = pending_loads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (static_cast<uint32_t>(i) < n) {
            e[i].map = p[i].map, e[i].dst = p[i].dst, e[i].x = p[i].x, e[i].y = p[i].y, e[i].shape = p[i].shape;
        }
    }
    issue_copies(bar, e, n);
    *count = 0;
}
// is there a TLOAD whose copy has not been issued yet?
__device__ __forceinline__ bool loads_pending()
{
    if (control()->mode & kModeEngineLoads) {
        volatile uint32_t *c = load_ring_counters();
        return c[1] != c[2];
    }
    return *pending_count() != 0;
}

// ---- tcgen05 helpers
__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// Block prologue / epilogue (called by the launch trampoline, not by tile programs).
__device__ __forceinline__ void block_begin(unsigned long long wait_limit_ns, uint32_t l0a_offset, uint32_t l0b_offset,
                                            int mode, uint32_t store_staging, const TmaTable *table)
{
    Control *ctl = control();
    const int nthreads = blockDim.x;
    for (int f = threadIdx.x; f < kNumFlags; f += nthreads) {
        // a flag raised by the matrix pipe is signalled by one tcgen05.commit; every other pipe's work is
        // done by all threads, so all of them arrive
        const int src = f / (kNumPipes * EVENT_ID_MAX), dst = (f / EVENT_ID_MAX) % kNumPipes;
        if (src == dst) {
            // no flags of a pipe with itself: PIPE_S -> PIPE_S holds the tile allocator's counters (tile_auto_place),
            // PIPE_V -> PIPE_V the flags held back for views (held_back)
            ctl->flags[f] = 0;
        } else if (kPipeWarps) {
            // the threads of the source pipe's team arrive; team B signals through one thread or the tensor core
            mbar_init(&ctl->flags[f], team_of_pipe(src) == kTeamC ? static_cast<uint32_t>(kTeamCThreads) : 1u);
        } else {
            mbar_init(&ctl->flags[f], src == PIPE_M ? 1u : static_cast<uint32_t>(nthreads));
        }
    }
    if ((threadIdx.x & 31) == 0) {
        for (int w = 0; w < kNumFlags / 32; ++w) {
            ctl->phase[w][threadIdx.x >> 5] = 0;
        }
    }
    for (int i = threadIdx.x; i < kWarps * kNumPipes * kNumPipes / 8; i += nthreads) {
        (&ctl->event_next[0][0])[i] = 0;
    }
    if (threadIdx.x < kNumDevFlags) {
        ctl->dev_flags[threadIdx.x] = 0;
    }
    for (int f = threadIdx.x; f < kNumFlags; f += nthreads) {
        ctl->raised[f] = 0;
        ctl->consumed[f] = 0;
    }
    if (threadIdx.x < kWarps) {
        ctl->core_static_init[threadIdx.x] = 0;
    }
    if (threadIdx.x == 0) {
        ctl->abort_flag = 0;
        ctl->mode = mode;
        ctl->fail_where = -1;
        ctl->wait_limit_ns = wait_limit_ns == 0 ? kWaitLimitNs : wait_limit_ns;
        ctl->l0a_offset = l0a_offset;
        ctl->l0b_offset = l0b_offset;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads(); // (the flag words of a pipe with itself were zeroed above)
    if (threadIdx.x == 0) {
        held_back()[13] = store_staging == kNoStoreStaging ? 0u : store_staging + 1u;
        tma_table() = table;
        load_ring_counters()[0] = 0;
        load_ring_counters()[1] = 0;
        load_ring_counters()[2] = 0;
        RegionBounds *rb = region_bounds();
        RegionShapes *rs = region_shapes();
        rs->count = 0;
        for (int r = 0; r < table->count && r < kMaxTmaRegions; ++r) {
            // (pitches of 4 GiB and more are left to the cp.async path)
            if (table->pitch_bytes[r] < (1ull << 32)) {
                const uint32_t i = rs->count;
                rb->base[i] = table->base[r];
                rb->end[i] = table->base[r] + table->bytes[r];
                rs->pitch_bytes[i] = static_cast<uint32_t>(table->pitch_bytes[r]);
                rs->row_bytes[i] = static_cast<uint32_t>(table->row_bytes[r]);
                rs->box_rows[i] = static_cast<uint16_t>(table->box_rows[r]);
                rs->elem_bytes[i] = static_cast<uint8_t>(table->elem_bytes[r]);
                region_reciprocals()[i] = static_cast<uint32_t>((1ull << 32) / table->pitch_bytes[r]);
                rs->count = i + 1;
            } else {
                break; // keeps cache index == table index
            }
        }
    }
    if ((threadIdx.x >> 5) == (kPipeWarps ? kTmemWarp : 0)) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                     "r"((mode >> kModeTmemColsShift) & 0x3ff)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
}

// pipe_warps: the loading thread brings its loads to completion (those prepared for the copy engine and not yet
// issued); the flag PIPE_MTE2 -> PIPE_ALL, 7 is kept for this
__device__ __noinline__ void complete_loads()
{
    if (!kPipeWarps || threadIdx.x != 0 || !loads_pending()) {
        return;
    }
    Control *ctl = control();
    const int f = flag_index(PIPE_MTE2, PIPE_ALL, 7);
    issue_pending_loads(&ctl->flags[f]);
    mbar_arrive(&ctl->flags[f]);
    volatile uint32_t *word = &ctl->phase[f >> 5][0];
    const uint32_t bit = 1u << (f & 31);
    const uint32_t w = *word;
    mbar_wait(&ctl->flags[f], (w & bit) ? 1u : 0u, f);
    *word = w ^ bit;
}

__device__ __forceinline__ void block_end(StatusRecord *status)
{
    complete_loads();
    asm volatile("cp.async.wait_all;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); // bulk stores of TSTORE have read their staging and landed
    tc_fence_before();
    __syncthreads();
    Control *ctl = control();
    if (ctl->abort_flag && threadIdx.x == 0 && status != nullptr) {
        if (atomicCAS(&status->code, 0, 4) == 0) { // a bounded wait gave up; the first block to report wins
            const int where = ctl->fail_where;
            status->block = static_cast<int>(blockIdx.x);
            status->where = where;
            status->detail = where >= 0 && where < kNumFlags ? ((where >> 6) & 7) * 16 + ((where >> 3) & 7) : -1;
            __threadfence();
        }
    }
    if ((threadIdx.x >> 5) == (kPipeWarps ? kTmemWarp : 0)) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(ctl->tmem_base),
                     "r"((ctl->mode >> kModeTmemColsShift) & 0x3ff)
                     : "memory");
    }
}
#endif // PTO_B200_DEVICE_CODE

// The real kernel that hosts a tile program.  It is declared here, before `__global__` loses its CUDA
// meaning for the rest of the translation unit (see pto-inst.hpp).
// What a launch may set beside the program: `status` is a device record (four ints, zero before the launch) that
// receives {4, block, flag, pipes} when a block gave up on a wait; `wait_limit_ns` bounds every wait of the program
// (0: two seconds); the two offsets place the Left and Right windows of the arena.
struct LaunchOptions {
    void *status = nullptr;
    int smem_bytes = kDefaultSmemBytes;
    unsigned long long wait_limit_ns = 0;
    uint32_t l0a_offset = PTO_B200_L0A_OFFSET;
    uint32_t l0b_offset = PTO_B200_L0B_OFFSET;
    // Every instruction completes before the next one starts, as in the reference's CPU simulation.  For tile programs
    // written for the simulation alone, which carry no set_flag / wait_flag between dependent instructions of
    // different pipes (e.g. RunTMATMUL_SPLIT_K of tests/cpu/st/testcase/tmatmul/tmatmul_kernel.cpp:104-155 in the
    // reference); programs that carry their flags do not need it and lose their overlap with it.
    bool in_order = false;
    // The core's pipes on warps of their own (kModePipeWarps above): loads, products and stores of a program that
    // orders its pipes with set_flag / wait_flag overlap as they do on the NPU.  For programs of one core's pipes
    // (no cross-core flags or TPipe rings); not together with in_order.
    bool pipe_warps = false;
    // TEXTRACT / TMOV (Mat -> Left / Right) of a window that starts on a 128-byte block of the contiguous dimension and
    // on a multiple of eight lines, and lies inside the staged tile, hands out a view instead of copying (the tensor
    // core reads any such window through its descriptor).  The flag that frees the staged tile for the next load is
    // then raised when the products that read the view are complete (see held_back).  Needs pipe_warps, and a
    // program that does not extract from a reloaded staged tile before the products of the previous one are issued.
    bool extract_views = false;
    // Arena offset (bytes, a multiple of 16) of kStoreStagingBytes (18 KiB) that the program's tiles leave free: TSTORE of
    // a whole fp32 accumulator tile to 16-byte aligned rows then goes through it, each thread staging 128 bytes of
    // its row and handing them to an asynchronous bulk copy, instead of storing 16 bytes per instruction.
    uint32_t store_staging_offset = kNoStoreStaging;
    // matrices whose tiles TLOAD may fetch with the copy engine (see TmaRegion)
    TmaRegion tma[kMaxTmaRegions];
    int tma_count = 0;
    // Every TLOAD of the program is a whole tile of a registered matrix (the launch gives up with {4, block, 601} if one
    // is not): the copies are then prepared ahead of time by a thread of their own (see load_ring), and the loading
    // thread only counts TLOADs and issues the prepared copies.  Needs pipe_warps and a registered matrix.
    bool engine_loads = false;
    // Tensor-memory columns the block allocates (a power of two from 32 to 512: accumulator tiles live below it).  With
    // 256 and at most half of the shared memory, two blocks share an SM (launch_two_per_sm): what one block's scalar
    // threads leave idle, the other block's use.
    int tmem_cols = kTmemCols;
};

// encodes the launch's registered matrices (host)
inline cudaError_t make_tma_table(const LaunchOptions &opt, TmaTable &table)
{
    memset(&table, 0, sizeof(table));
    if (opt.tma_count == 0) {
        return cudaSuccess;
    }
    if (opt.tma_count < 0 || opt.tma_count > kMaxTmaRegions) {
        return cudaErrorInvalidValue;
    }
    using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || fn == nullptr) {
        return cudaErrorNotSupported;
    }
    for (int i = 0; i < opt.tma_count; ++i) {
        const TmaRegion &r = opt.tma[i];
        const uint64_t es = static_cast<uint64_t>(r.elem_bytes);
        if (r.base == nullptr || (es != 1 && es != 2) || r.box_rows == 0 || r.box_rows > 256 ||
            (r.box_rows & (r.box_rows - 1)) != 0 || r.rows == 0 || r.cols == 0 ||
            (reinterpret_cast<uintptr_t>(r.base) & 15u) != 0 || ((r.pitch * es) & 15u) != 0 || r.pitch < r.cols) {
            return cudaErrorInvalidValue;
        }
        const cuuint64_t dims[2] = {r.cols, r.rows};
        const cuuint64_t strides[1] = {r.pitch * es};
        const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / es), r.box_rows};
        const cuuint32_t elem_strides[2] = {1, 1};
        if (reinterpret_cast<EncodeFn>(fn)(&table.map[i], es == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                                           const_cast<void *>(r.base), dims, strides, box, elem_strides,
                                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            return cudaErrorInvalidValue;
        }
        table.base[i] = reinterpret_cast<unsigned long long>(r.base);
        table.bytes[i] = ((r.rows - 1) * r.pitch + r.cols) * es;
        table.pitch_bytes[i] = r.pitch * es;
        table.row_bytes[i] = r.cols * es;
        table.box_rows[i] = r.box_rows;
        table.elem_bytes[i] = static_cast<uint32_t>(es);
    }
    table.count = opt.tma_count;
    return cudaSuccess;
}

template <typename Program, int kBlocksPerSm = 1>
__global__ void __launch_bounds__(kBlockThreads, kBlocksPerSm)
    block_kernel(Program program, StatusRecord *status, unsigned long long wait_limit_ns, uint32_t l0a_offset,
                 uint32_t l0b_offset, int mode, uint32_t store_staging, const __grid_constant__ TmaTable tma)
{
#if PTO_B200_DEVICE_CODE
    if ((smem_u32(smem_base()) & 1023u) != 0) {
        if (threadIdx.x == 0 && status != nullptr && atomicCAS(&status->code, 0, 3) == 0) {
            status->block = static_cast<int>(blockIdx.x);
            status->where = -3; // the shared-memory buffer is not 1 KiB aligned
            status->detail = static_cast<int>(smem_u32(smem_base()) & 1023u);
        }
        return;
    }
    block_begin(wait_limit_ns, l0a_offset, l0b_offset, mode, store_staging, &tma);
    if (kPipeWarps && (threadIdx.x & 31) != 0 &&
        ((threadIdx.x >> 5) == 0 || (threadIdx.x >> 5) == kTeamBWarp || ((mode & kModeEngineLoads) && (threadIdx.x >> 5) == 1))) {
        return; // the loading thread, the thread of MTE1 / M (and the preparing thread) work alone in their warps
    }
    program();
    block_end(status);
#endif
}

// Launches `program` (a __device__ callable) on `blocks` thread blocks of the stream.
template <int kBlocksPerSm, typename Program>
inline cudaError_t launch_impl(uint32_t blocks, void *stream, Program program, const LaunchOptions &opt)
{
    if (opt.pipe_warps != kPipeWarps || (opt.pipe_warps && opt.in_order)) {
        return cudaErrorInvalidValue; // pipe_warps is compiled in (PTO_B200_PIPE_WARPS) and excludes in_order
    }
    if (opt.tmem_cols < 32 || opt.tmem_cols > kTmemCols || (opt.tmem_cols & (opt.tmem_cols - 1)) != 0 ||
        opt.smem_bytes <= kControlBytes || opt.smem_bytes > kDefaultSmemBytes) {
        return cudaErrorInvalidValue;
    }
    TmaTable table;
    cudaError_t e = make_tma_table(opt, table);
    if (e != cudaSuccess) {
        return e;
    }
    auto kernel = block_kernel<Program, kBlocksPerSm>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, opt.smem_bytes);
    if (e != cudaSuccess) {
        return e;
    }
    if (kBlocksPerSm > 1) {
        // the whole of the SM's shared memory, so that two blocks fit side by side
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) {
            return e;
        }
    }
    kernel<<<blocks, kBlockThreads, opt.smem_bytes, static_cast<cudaStream_t>(stream)>>>(
        program, static_cast<StatusRecord *>(opt.status), opt.wait_limit_ns, opt.l0a_offset, opt.l0b_offset,
        (opt.in_order ? kModeInOrder : 0) | (kPipeWarps ? kModePipeWarps : 0) |
            (opt.pipe_warps && opt.extract_views ? kModeViews : 0) |
            (opt.pipe_warps && opt.engine_loads && opt.tma_count > 0 ? kModeEngineLoads : 0) |
            (opt.tmem_cols << kModeTmemColsShift),
        opt.store_staging_offset, table);
    return cudaGetLastError();
}
template <typename Program>
inline cudaError_t launch(uint32_t blocks, void *stream, Program program, const LaunchOptions &opt)
{
    return launch_impl<1>(blocks, stream, program, opt);
}
// The same with two blocks per SM: `opt.smem_bytes` at most half of an SM's shared memory (113 KiB) and
// `opt.tmem_cols` at most 256; the kernel is compiled for at most 128 registers per thread.
template <typename Program>
inline cudaError_t launch_two_per_sm(uint32_t blocks, void *stream, Program program, const LaunchOptions &opt)
{
    if (opt.smem_bytes > 113 * 1024 || opt.tmem_cols > 256) {
        return cudaErrorInvalidValue;
    }
    return launch_impl<2>(blocks, stream, program, opt);
}
template <typename Program>
inline cudaError_t launch(uint32_t blocks, void *stream, Program program, void *status = nullptr,
                          int smem_bytes = kDefaultSmemBytes)
{
    LaunchOptions opt;
    opt.status = status;
    opt.smem_bytes = smem_bytes;
    return launch(blocks, stream, program, opt);
}

} // namespace b200
} // namespace pto

// Launch statement for kernels written in the reference's style.  `kernel` is the parenthesised kernel
// name (with its template arguments), followed by the block count, the stream and the kernel's arguments.
#define PTO_B200_LAUNCH(kernel, blocks, stream, ...) \
    (void)pto::b200::launch((blocks), (stream), [=] __device__() { kernel(__VA_ARGS__); })

// start of the block's arena (the address space of Vec and Mat tiles) for programs that place data there themselves,
// e.g. the ring of an on-chip FIFO
PTO_INTERNAL uint8_t *pto_b200_arena()
{
#if PTO_B200_DEVICE_CODE
    return pto::b200::arena();
#else
    return nullptr;
#endif
}

// ---------------------------------------------------------------- block id, flags
PTO_INTERNAL uint32_t get_block_idx()
{
#if PTO_B200_DEVICE_CODE
    return blockIdx.x;
#else
    return 0;
#endif
}
PTO_INTERNAL uint32_t get_block_num()
{
#if PTO_B200_DEVICE_CODE
    return gridDim.x;
#else
    return 1;
#endif
}

namespace pto {
namespace b200 {
// a pipe ordered with itself: the threads that run it meet
PTO_INTERNAL void pipe_self_barrier(pipe_t pipe)
{
#if PTO_B200_DEVICE_CODE
    if (!kPipeWarps) {
        __syncthreads();
        return;
    }
    const int team = team_of_pipe(pipe);
    if (team == kTeamL) {
        sync_l();
    } else if (team == kTeamC) {
        sync();
    }
#else
    (void)pipe;
#endif
}
} // namespace b200
} // namespace pto

// set_flag(src, dst, id): the flag is raised once everything issued so far on pipe `src` is complete.
//   PIPE_M    : tcgen05.commit by the issuing thread (covers all earlier tcgen05.mma)
//   PIPE_MTE2 : every thread arrives when its own asynchronous copies have landed
//   others    : their work is synchronous per thread, every thread arrives
// With PTO_B200_PIPE_WARPS the threads of `src` raise the flag (one thread for MTE2, MTE1 and M, the four warps of
// team C for the rest), and a flag between two teams is raised again only when its previous raise has been consumed
// (Control::raised).
namespace pto {
namespace b200 {
#if PTO_B200_DEVICE_CODE
// the count of raises of a flag between teams, advanced by the one thread that raises it
__device__ __forceinline__ void next_raise(Control *ctl, int f)
{
    const uint8_t n = *reinterpret_cast<volatile uint8_t *>(&ctl->raised[f]);
    wait_until_consumed(f, n);
    ctl->raised[f] = static_cast<uint8_t>(n + 1);
}
__device__ __forceinline__ void set_flag_pipe_warps(pipe_t src, pipe_t dst, int id)
{
    if (!runs(src)) {
        return;
    }
    Control *ctl = control();
    const int f = flag_index(src, dst, id);
    uint64_t *bar = &ctl->flags[f];
    stamp(0x3000 + f);
    const int team = team_of_pipe(src);
    const bool between_teams = team != team_of_pipe(dst);
    volatile uint32_t *held = held_back();
    if (src == PIPE_M) {
        if (between_teams) {
            next_raise(ctl, f);
        }
        tc_commit(bar);
        // flags held back for views: the products that read them are all issued by now
        const uint32_t count = held[0];
        for (uint32_t i = 0; i < count; ++i) {
            const int hf = static_cast<int>(held[1 + i]);
            next_raise(ctl, hf);
            tc_commit(&ctl->flags[hf]);
        }
        if (count != 0) {
            held[0] = 0;
        }
        held[15] = 0;
    } else if (src == PIPE_MTE1) {
        if (!between_teams) {
            // MTE1 -> M: the same thread stages operands and issues products, program order is the order; copies
            // made through the generic proxy are made visible to the tensor core
            if (held[14] != 0) {
                fence_async_proxy();
            }
        } else if (dst == PIPE_MTE2 && held[15] != 0 && held[0] < kMaxHeldBack) {
            // a view was handed out since the matrix pipe last raised a flag: held back (see held_back)
            held[1 + held[0]] = static_cast<uint32_t>(f);
            held[0] = held[0] + 1;
        } else {
            if (held[14] != 0) {
                fence_async_proxy();
            }
            next_raise(ctl, f);
            mbar_arrive(bar);
        }
    } else if (src == PIPE_MTE2) {
        // thread 0: the copy engine's loads of the TLOADs before this flag complete on it; tiles copied by the
        // helping threads were complete when their TLOAD returned
        // The copies are issued as soon as the flag's previous phase is complete (their bytes then count for this
        // one), which is well before the previous raise has been consumed: the data is on its way while the loading
        // thread waits for the consumer; the arrival that completes the phase comes after that wait.
        const uint8_t n = *reinterpret_cast<volatile uint8_t *>(&ctl->raised[f]);
        const bool consumed = *reinterpret_cast<volatile uint8_t *>(&ctl->consumed[f]) == n;
        if (loads_pending()) {
            if (!consumed) {
                mbar_wait(bar, (static_cast<uint32_t>(n) + 1u) & 1u, f); // phase n - 1 (a fresh barrier passes)
            }
            issue_pending_loads(bar);
        }
        if (between_teams) {
            if (!consumed) {
                wait_until_consumed(f, n);
            }
            ctl->raised[f] = static_cast<uint8_t>(n + 1);
        }
        if (held[14] != 0) {
            fence_async_proxy();
        }
        mbar_arrive(bar);
    } else {
        // team C: every thread of the four warps arrives; the first one keeps the count
        if (between_teams) {
            sync();
            const uint8_t n = *reinterpret_cast<volatile uint8_t *>(&ctl->raised[f]);
            sync();
            if (static_cast<int>(threadIdx.x) == team_first_thread(kTeamC)) {
                ctl->raised[f] = static_cast<uint8_t>(n + 1);
            }
            wait_until_consumed(f, n);
        }
        fence_async_proxy();
        tc_fence_before();
        mbar_arrive(bar);
    }
    stamp(0x3800 + f);
}
#endif
} // namespace b200
} // namespace pto

PTO_INTERNAL void set_flag(pipe_t src, pipe_t dst, int id)
{
#if PTO_B200_DEVICE_CODE
    if (src == dst) {
        pto::b200::pipe_self_barrier(src); // a pipe is ordered with itself by a barrier, not a flag
        return;
    }
    if constexpr (pto::b200::kPipeWarps) {
        pto::b200::set_flag_pipe_warps(src, dst, id);
        return;
    }
    pto::b200::Control *ctl = pto::b200::control();
    const int f = pto::b200::flag_index(src, dst, id);
    uint64_t *bar = &ctl->flags[f];
    pto::b200::stamp(0x3000 + f);
    if (src == PIPE_M) {
        if (threadIdx.x == 0) {
            pto::b200::tc_commit(bar);
        }
    } else if (src == PIPE_MTE2) {
        pto::b200::mbar_arrive_after_copies(bar);
    } else {
        // shared-memory writes of this thread become visible to the tensor core's (asynchronous-proxy) reads
        pto::b200::fence_async_proxy();
        pto::b200::tc_fence_before();
        pto::b200::mbar_arrive(bar);
    }
    pto::b200::stamp(0x3800 + f);
#else
    (void)src;
    (void)dst;
    (void)id;
#endif
}

// wait_flag(src, dst, id): every thread waits for the matching set_flag (the n-th wait pairs with the n-th set).
namespace pto {
namespace b200 {
#if PTO_B200_DEVICE_CODE
__device__ __forceinline__ void wait_flag_pipe_warps(pipe_t src, pipe_t dst, int id)
{
    if (!runs(dst)) {
        return; // the threads of the waiting pipe wait
    }
    const int team = team_of_pipe(dst);
    const bool between_teams = team_of_pipe(src) != team;
    if (team == kTeamB && !between_teams && src == PIPE_MTE1) {
        return; // MTE1 -> M on one thread: see set_flag
    }
    Control *ctl = control();
    const int f = flag_index(src, dst, id);
    stamp(0x1000 + f);
    if (team != kTeamC) {
        // one thread waits.  Between teams the count of completed waits is also the phase
        if (between_teams) {
            const uint8_t done = *reinterpret_cast<volatile uint8_t *>(&ctl->consumed[f]);
            if (mbar_wait(&ctl->flags[f], done & 1u, f)) {
                ctl->consumed[f] = static_cast<uint8_t>(done + 1);
            }
        } else {
            volatile uint32_t *word = &ctl->phase[f >> 5][threadIdx.x >> 5];
            const uint32_t bit = 1u << (f & 31);
            const uint32_t w = *word;
            mbar_wait(&ctl->flags[f], (w & bit) ? 1u : 0u, f);
            *word = w ^ bit;
        }
        if (held_back()[14] != 0) {
            fence_async_proxy(); // tiles written through the generic proxy, read by the tensor core
        }
    } else {
        volatile uint32_t *word = &ctl->phase[f >> 5][threadIdx.x >> 5];
        const uint32_t bit = 1u << (f & 31);
        const uint32_t parity = (*word & bit) ? 1u : 0u;
        const bool ok = mbar_wait(&ctl->flags[f], parity, f);
        __syncwarp();
        if ((threadIdx.x & 31) == 0) {
            *word = *word ^ bit;
        }
        __syncwarp();
        if (between_teams) {
            // every warp of the team is past the wait: the flag may be raised again (Control::consumed)
            sync();
            if (ok && static_cast<int>(threadIdx.x) == team_first_thread(kTeamC)) {
                ctl->consumed[f] = static_cast<uint8_t>(ctl->consumed[f] + 1);
            }
        }
        fence_async_proxy();
    }
    tc_fence_after();
    stamp(0x2000 + f);
}
#endif
} // namespace b200
} // namespace pto

PTO_INTERNAL void wait_flag(pipe_t src, pipe_t dst, int id)
{
#if PTO_B200_DEVICE_CODE
    if (src == dst) {
        return; // see set_flag
    }
    if constexpr (pto::b200::kPipeWarps) {
        pto::b200::wait_flag_pipe_warps(src, dst, id);
        return;
    }
    pto::b200::Control *ctl = pto::b200::control();
    const int f = pto::b200::flag_index(src, dst, id);
    pto::b200::stamp(0x1000 + f);
    // all lanes of a warp run the same instruction stream, so the phase is kept once per warp
    volatile uint32_t *word = &ctl->phase[f >> 5][threadIdx.x >> 5];
    const uint32_t bit = 1u << (f & 31);
    const uint32_t parity = (*word & bit) ? 1u : 0u;
    pto::b200::mbar_wait(&ctl->flags[f], parity, f);
    __syncwarp();
    if ((threadIdx.x & 31) == 0) {
        *word = *word ^ bit;
    }
    __syncwarp();
    pto::b200::tc_fence_after();
    pto::b200::fence_async_proxy();
    pto::b200::stamp(0x2000 + f);
#else
    (void)src;
    (void)dst;
    (void)id;
#endif
}

namespace pto {
namespace b200 {
// in-order launches: what an asynchronous instruction does before it returns
PTO_INTERNAL void complete_copies_if_in_order()
{
#if PTO_B200_DEVICE_CODE
    if (!kPipeWarps && (control()->mode & kModeInOrder)) {
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
    }
#endif
}
PTO_INTERNAL void complete_matmul_if_in_order()
{
#if PTO_B200_DEVICE_CODE
    if (!kPipeWarps && (control()->mode & kModeInOrder)) {
        // the flag (PIPE_M -> PIPE_ALL, 7) is kept for this; tile programs have no reason to name it
        set_flag(PIPE_M, PIPE_ALL, 7);
        wait_flag(PIPE_M, PIPE_ALL, 7);
        __syncthreads();
    }
#endif
}
} // namespace b200
} // namespace pto

PTO_INTERNAL void pipe_barrier(pipe_t pipe)
{
#if PTO_B200_DEVICE_CODE
    if (!pto::b200::pipe_warps()) {
        __syncthreads();
        return;
    }
    if (pipe == PIPE_ALL) {
        // every pipe drains what it has in flight: the loads of MTE2, the products of M (awaited by the warps of the
        // vector and store pipes, which then meet)
        pto::b200::complete_loads();
        set_flag(PIPE_M, PIPE_ALL, 7);
        wait_flag(PIPE_M, PIPE_ALL, 7);
        pto::b200::sync();
    } else if (pipe == PIPE_MTE2) {
        pto::b200::complete_loads();
    } else {
        pto::b200::pipe_self_barrier(pipe);
    }
#else
    (void)pipe;
#endif
}

// ---------------------------------------------------------------- cross-core flags
// On the NPU the cube core and the two vector cores of an AI core signal each other through FFTS flags
// (include/pto/npu/a2a3/TPush.hpp:141-162 in the reference: ffts_cross_core_sync raises flag `id` once everything
// issued so far on `pipe` is complete, wait_flag_dev(id) consumes one raise).  Here one thread block plays both roles
// in program order, so a flag is a counter in the control block: the raise happens after the block's outstanding
// copies and stores are complete, the wait is bounded like every other wait.
#if PTO_B200_DEVICE_CODE
namespace pto {
namespace b200 {
// pipe_warps: a cross-core flag is a count of raises (Control::dev_flags, never decremented) and, per team, a count of
// the raises it has seen (flag words of PIPE_MTE1 -> PIPE_MTE1, behind the timeline's counters).  The core's scalar unit
// stalls at wait_flag_dev on the NPU; here every team walks the instruction stream, so every team waits there, each
// against its own count.
__device__ __forceinline__ volatile uint8_t *dev_flags_seen(int team)
{
    return reinterpret_cast<volatile uint8_t *>(&control()->flags[flag_index(PIPE_MTE1, PIPE_MTE1, 0)]) + 12 + team * kNumDevFlags;
}
static_assert(12 + 3 * kNumDevFlags <= 64, "three teams' counts fit the eight flag words");
// the team whose flags and cross-core waits this thread executes (-1: none)
__device__ __forceinline__ int my_team()
{
    if (threadIdx.x == 0) {
        return kTeamL;
    }
    if (threadIdx.x == kTeamBWarp * 32) {
        return kTeamB;
    }
    return threadIdx.x >= kTeamCFirstWarp * 32 ? kTeamC : -1;
}
__device__ __noinline__ void raise_dev_flag_pipe_warps(pipe_t pipe, int id)
{
    if (!runs(pipe)) {
        return;
    }
    Control *ctl = control();
    const int team = team_of_pipe(pipe);
    // everything issued so far on the pipe is complete, and visible to the other teams, before the raise
    if (team == kTeamL) {
        complete_loads();
        __threadfence();
        atomicAdd(&ctl->dev_flags[id], 1);
    } else if (team == kTeamB) {
        if (pipe == PIPE_M) {
            set_flag(PIPE_M, PIPE_MTE1, 7); // (PIPE_M -> PIPE_MTE1, 7 is kept for this: the products are complete)
            wait_flag(PIPE_M, PIPE_MTE1, 7);
        }
        __threadfence();
        atomicAdd(&ctl->dev_flags[id], 1);
    } else {
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); // staged stores of TSTORE have landed
        __threadfence();
        sync();
        if (static_cast<int>(threadIdx.x) == team_first_thread(kTeamC)) {
            atomicAdd(&ctl->dev_flags[id], 1);
        }
    }
}
__device__ __noinline__ void wait_dev_flag_pipe_warps(int id)
{
    const int team = my_team();
    if (team < 0) {
        return;
    }
    Control *ctl = control();
    volatile uint8_t *seen = dev_flags_seen(team) + id;
    const uint8_t have = *seen;
    volatile int *flag = &ctl->dev_flags[id];
    volatile int *abort_flag = &ctl->abort_flag;
    unsigned long long t0 = 0;
    for (uint32_t i = 0; static_cast<uint8_t>(static_cast<uint8_t>(*flag) - have) == 0; ++i) {
        if ((i & 0x3f) == 0x3f) {
            if (*abort_flag) {
                break;
            }
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > ctl->wait_limit_ns) {
                give_up(kNumFlags + id);
                break;
            }
        }
    }
    if (team == kTeamC) {
        sync(); // every thread of the team has read its count
        if (static_cast<int>(threadIdx.x) == team_first_thread(kTeamC)) {
            *seen = static_cast<uint8_t>(have + 1);
        }
        sync();
    } else {
        *seen = static_cast<uint8_t>(have + 1);
    }
    __threadfence();
    if (held_back()[14] != 0) {
        fence_async_proxy();
    }
}
} // namespace b200
} // namespace pto
#endif

PTO_INTERNAL void ffts_cross_core_sync(pipe_t pipe, uint64_t config)
{
#if PTO_B200_DEVICE_CODE
    if constexpr (pto::b200::kPipeWarps) {
        pto::b200::raise_dev_flag_pipe_warps(pipe, static_cast<int>((config >> 8) & 0xf));
        return;
    }
    (void)pipe;
    const int id = static_cast<int>((config >> 8) & 0xf);
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads(); // global and shared-memory writes of every thread are visible to the block from here on
    if (threadIdx.x == 0) {
        atomicAdd(&pto::b200::control()->dev_flags[id], 1);
    }
    __syncthreads();
#else
    (void)pipe;
    (void)config;
#endif
}

PTO_INTERNAL void wait_flag_dev(int id)
{
#if PTO_B200_DEVICE_CODE
    if constexpr (pto::b200::kPipeWarps) {
        pto::b200::wait_dev_flag_pipe_warps(id & 0xf);
        return;
    }
    pto::b200::Control *ctl = pto::b200::control();
    volatile int *flag = &ctl->dev_flags[id & 0xf];
    volatile int *abort_flag = &ctl->abort_flag;
    __syncthreads();
    unsigned long long t0 = 0;
    for (uint32_t i = 0; *flag <= 0; ++i) {
        if ((i & 0x3f) == 0x3f) {
            if (*abort_flag) {
                break;
            }
            const unsigned long long now = pto::b200::global_timer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > ctl->wait_limit_ns) {
                pto::b200::give_up(pto::b200::kNumFlags + (id & 0xf));
                break;
            }
            __nanosleep(64);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && *flag > 0) {
        atomicSub(&ctl->dev_flags[id & 0xf], 1);
    }
    __syncthreads();
#else
    (void)id;
#endif
}
PTO_INTERNAL void set_ffts_base_addr(uint64_t) {}
// the NPU's system counter (the reference's kernels stamp their start and end with it): nanoseconds of the global timer
PTO_INTERNAL uint64_t get_sys_cnt()
{
#if PTO_B200_DEVICE_CODE
    return pto::b200::global_timer_ns();
#else
    return 0;
#endif
}
// one block hosts the cube role and a single vector role
PTO_INTERNAL uint32_t get_subblockid() { return 0; }
PTO_INTERNAL uint32_t get_subblockdim() { return 1; }

namespace pto {
namespace b200 {

// ---------------------------------------------------------------- function-local statics of tile programs
// A `static` local in a device function is ONE variable for the whole grid in CUDA, where the reference's kernels
// expect one per core (its instruction stream is scalar there).  PTO_B200_CORE_STATIC(T, name, init, slot) declares
// the per-core replacement: the value lives in the block's control area, one copy per warp (every lane of a warp runs
// the same scalar stream); reads and writes go through this proxy, which keeps the lanes of a warp in step.
template <typename T, int Slot>
struct CoreStatic {
    static_assert(Slot >= 0 && Slot < kNumCoreStatics, "PTO_B200_CORE_STATIC: slot out of range");
    static_assert(sizeof(T) <= 8 && std::is_integral_v<T>, "PTO_B200_CORE_STATIC: integral types of up to 8 bytes");
#if PTO_B200_DEVICE_CODE
    __device__ __forceinline__ explicit CoreStatic(T init)
    {
        Control *c = control();
        const int warp = threadIdx.x >> 5;
        __syncwarp();
        const bool have = (c->core_static_init[warp] >> Slot) & 1u;
        __syncwarp();
        if (!have && (threadIdx.x & 31) == 0) {
            c->core_static[Slot][warp] = static_cast<unsigned long long>(init);
            c->core_static_init[warp] |= 1u << Slot;
        }
        __syncwarp();
    }
    __device__ __forceinline__ T get() const
    {
        __syncwarp();
        const T v = static_cast<T>(control()->core_static[Slot][threadIdx.x >> 5]);
        __syncwarp();
        return v;
    }
    __device__ __forceinline__ void set(T v)
    {
        __syncwarp();
        if ((threadIdx.x & 31) == 0) {
            control()->core_static[Slot][threadIdx.x >> 5] = static_cast<unsigned long long>(v);
        }
        __syncwarp();
    }
#else
    explicit CoreStatic(T init) : host_(init) {}
    T get() const { return host_; }
    void set(T v) { host_ = v; }
    T host_;
#endif
    PTO_INTERNAL operator T() const { return get(); }
    PTO_INTERNAL CoreStatic &operator=(T v)
    {
        set(v);
        return *this;
    }
    PTO_INTERNAL CoreStatic &operator^=(T v) { return *this = static_cast<T>(get() ^ v); }
    PTO_INTERNAL CoreStatic &operator+=(T v) { return *this = static_cast<T>(get() + v); }
    PTO_INTERNAL CoreStatic &operator-=(T v) { return *this = static_cast<T>(get() - v); }
};

// next automatic event id of a (source pipe, destination pipe) pair, ids 0..7 in turn
// (include/pto/common/event.hpp:112-135 in the reference keeps this counter in a function-local static)
PTO_INTERNAL event_t next_event_id(pipe_t src, pipe_t dst)
{
#if PTO_B200_DEVICE_CODE
    Control *c = control();
    const int pair = (src & 7) * kNumPipes + (dst & 7);
    uint32_t *word = &c->event_next[threadIdx.x >> 5][pair >> 3];
    const int shift = (pair & 7) * 4;
    __syncwarp();
    const uint32_t w = *word;
    __syncwarp();
    const uint32_t id = (w >> shift) & 0xfu;
    if ((threadIdx.x & 31) == 0) {
        *word = (w & ~(0xfu << shift)) | (((id + 1) % EVENT_ID_MAX) << shift);
    }
    __syncwarp();
    return static_cast<event_t>(id);
#else
    (void)src;
    (void)dst;
    return EVENT_ID0;
#endif
}

} // namespace b200
} // namespace pto

#define PTO_B200_CORE_STATIC(T, name, init, slot) pto::b200::CoreStatic<T, slot> name(static_cast<T>(init))
