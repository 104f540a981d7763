// TPUSH / TPOP / TFREE and the FIFO pipes between the cube role and the vector role of a core.
// Interface: include/pto/common/fifo.hpp:20-83 (DataFIFO, FIFOType, VecCubeRatio), include/pto/common/pto_instr.hpp:
// 1434-1474 (TPUSH / TPOP / TFREE), include/pto/npu/a2a3/TPush.hpp:21-388 and TPop.hpp:26-58 (TSyncOpType, TPipe with
// its Producer / Consumer and their status setters), include/pto/cpu/TPush.hpp:21-133 (TFIFOSync, the simulation's
// producer / consumer pair) - paths relative to the reference root.
//
// On the NPU a pipe carries tiles between two cores through a ring of entries in global memory, with FFTS flags for
// "entry filled" (FlagID) and "entry free again" (FlagID + 1).  On this backend one thread block plays both roles, so:
//   * the ring may live in global memory (FIFOType::GM_FIFO, the caller's workspace, as in the reference) or in the
//     block's shared-memory arena (VEC_FIFO / MAT_FIFO: the pointer given to the pipe is a tile's data()); entries are
//     written by TSTORE's code path and read by TLOAD's, both of which take either kind of address;
//   * the two flags are the block's cross-core counters (runtime.hpp: ffts_cross_core_sync / wait_flag_dev), every
//     wait bounded.
// An entry holds the consumer's view of the data: a producer tile wider than the consumer's is stored as consecutive
// consumer-width slabs, a consumer tile wider than the producer's is assembled from consecutive producer-width slabs,
// exactly as the reference lays its entries out (TPush.hpp:160-200, 296-330).
#pragma once

#include "instr.hpp"

namespace pto {

enum class FIFOType : uint8_t {
    GM_FIFO = 0,  // ring in global memory
    VEC_FIFO = 1, // ring in the vector role's local memory
    MAT_FIFO = 2, // ring in the cube role's local memory
};

enum class VecCubeRatio : uint8_t {
    V1C1_VEC0 = 0,
    V1C1_VEC1 = 1,
    V2C1_VECS = 2,
};

template <typename DataType, FIFOType FifoType, int Depth, int Period>
struct DataFIFO {
    static constexpr int fifoDepth = Depth;
    static constexpr int fifoPeriod = Period;
    static constexpr FIFOType fifoType = FifoType;
    using DType = DataType;

    DataType *fifoBase;

    PTO_INTERNAL DataFIFO(DataType *ptr) : fifoBase(ptr) {}
    PTO_INTERNAL DataType *getBasePtr() { return fifoBase; }
};

// what the producer does to fill an entry and the consumer to read it
enum class TSyncOpType : uint8_t {
    TSTORE_C2GM_UFON,  // accumulator store by the cube role (unit flag on)
    TSTORE_C2GM_UFOFF, // accumulator store by the cube role (unit flag off)
    TSTORE_C2GM,       // accumulator store by the cube role
    TSTORE_V2GM,       // vector-tile store by the vector role
    TMOV_C2UB,         // accumulator moved into the vector role's memory
    TINSERT_V2L1,      // vector tile inserted into the cube role's memory
    TLOAD,             // the consumer's load
};

enum TSyncCVMode : uint8_t { CUBE_ALL_CORE_SYNC = 0, VEC_ALL_CORE_SYNC = 0, VEC_SUBCORES_SYNC = 1, CV_CORES_SYNC = 2 };

template <TSyncOpType ProducerOp, TSyncOpType ConsumerOp>
struct TSyncTraits {
    static constexpr bool is_cube_to_vec =
        (ProducerOp == TSyncOpType::TSTORE_C2GM_UFON) || (ProducerOp == TSyncOpType::TSTORE_C2GM_UFOFF) ||
        (ProducerOp == TSyncOpType::TSTORE_C2GM) || (ProducerOp == TSyncOpType::TMOV_C2UB);
    static constexpr bool is_vec_to_cube =
        (ProducerOp == TSyncOpType::TSTORE_V2GM) || (ProducerOp == TSyncOpType::TINSERT_V2L1);
    static_assert(ConsumerOp == TSyncOpType::TLOAD, "Consumer operation must be TLOAD");
    static_assert(is_cube_to_vec || is_vec_to_cube, "Producer must be a cube-role or a vector-role store");
};

namespace b200 {

PTO_INTERNAL uint64_t ffts_config(uint16_t flag_id)
{
    return 0x1u | (static_cast<uint64_t>(CV_CORES_SYNC) << 4) | (static_cast<uint64_t>(flag_id & 0xf) << 8);
}

// rows x cols elements at `addr` with `pitch` elements between rows, as a global tensor TLOAD / TSTORE understand
template <typename T, int kRows, int kCols, int kPitch>
using EntryView = GlobalTensor<T, Shape<1, 1, 1, kRows, kCols>, Stride<1, 1, 1, kPitch, 1>>;

// producer side: `tile` into the entry at `addr` (consumer-width slabs of kConsM x kConsN elements)
template <typename T, int kConsM, int kConsN, typename TileProd>
PTO_INTERNAL void entry_store(T *addr, TileProd &tile)
{
    constexpr int kProdM = TileProd::Rows, kProdN = TileProd::Cols;
    if constexpr (TileProd::Loc == TileType::Acc) {
        // an accumulator of the producer's width; a wider consumer tile is made of kConsN / kProdN such entries in a row
        EntryView<T, kProdM, kProdN, kProdN> view(addr);
        TSTORE(view, tile);
    } else {
        static_assert(TileProd::Loc == TileType::Vec && TileProd::isRowMajor, "TPUSH: accumulator or row-major vector tiles");
        constexpr int kSlabs = (kProdN >= kConsN) ? kProdN / kConsN : 1;
        constexpr int kWidth = (kProdN >= kConsN) ? kConsN : kProdN;
        using Slab = Tile<TileType::Vec, T, kProdM, kProdN, BLayout::RowMajor, kProdM, kWidth>;
        for (int s = 0; s < kSlabs; ++s) {
            Slab slab;
            TASSIGN(slab, tile.data() + s * kWidth);
            EntryView<T, kProdM, kWidth, kWidth> view(addr + static_cast<size_t>(s) * kConsM * kConsN);
            TSTORE(view, slab);
        }
    }
}

// consumer side: the entry at `addr` into `tile`
template <typename T, int kProdM, int kProdN, typename TileCons>
PTO_INTERNAL void entry_load(T *addr, TileCons &tile)
{
    constexpr int kConsM = TileCons::Rows, kConsN = TileCons::Cols;
    if constexpr (TileCons::Loc == TileType::Mat) {
        EntryView<T, kConsM, kConsN, kConsN> view(addr);
        TLOAD(tile, view);
    } else {
        static_assert(TileCons::Loc == TileType::Vec && TileCons::isRowMajor, "TPOP: matrix or row-major vector tiles");
        constexpr int kSlabs = (kConsN >= kProdN) ? kConsN / kProdN : 1;
        constexpr int kWidth = (kConsN >= kProdN) ? kProdN : kConsN;
        using Slab = Tile<TileType::Vec, T, kConsM, kConsN, BLayout::RowMajor, kConsM, kWidth>;
        for (int s = 0; s < kSlabs; ++s) {
            Slab slab;
            TASSIGN(slab, tile.data() + s * kWidth);
            EntryView<T, kConsM, kWidth, kWidth> view(addr + static_cast<size_t>(s) * kProdM * kProdN);
            TLOAD(slab, view);
        }
    }
}

} // namespace b200

// ---------------------------------------------------------------- TPipe (the NPU kernels' pipe)
template <uint8_t FlagID, FIFOType FiFoType, uint8_t FiFoDepth, uint8_t FiFoSyncT, typename TileDataProd,
          typename TileDataCons, TSyncOpType ProducerOp, TSyncOpType ConsumerOp,
          VecCubeRatio VCRatio = VecCubeRatio::V2C1_VECS>
struct TPipe {
    using Traits = TSyncTraits<ProducerOp, ConsumerOp>;
    static constexpr bool is_c2v = Traits::is_cube_to_vec;
    static constexpr bool is_v2c = Traits::is_vec_to_cube;
    using T = typename TileDataCons::DType;
    static_assert(sizeof(T) == sizeof(typename TileDataProd::DType), "TPipe: producer and consumer element sizes differ");
    using DataFiFo = DataFIFO<T, FiFoType, FiFoDepth, FiFoSyncT>;

    // elements of one entry: the larger of the two tiles
    static constexpr int kProdElems = TileDataProd::Rows * TileDataProd::Cols;
    static constexpr int kConsElems = TileDataCons::Rows * TileDataCons::Cols;
    static constexpr int kEntryElems = kProdElems > kConsElems ? kProdElems : kConsElems;

    PTO_INTERNAL static uint64_t getFFTSMsgCfg(TSyncCVMode mode, uint16_t flagID, uint16_t base_const = 0x1)
    {
        return (base_const & 0xf) + ((mode & 0x3) << 4) + ((flagID & 0xf) << 8);
    }

    struct Producer {
        int tile_id = -1;
        int sub_tile_id = -1;
        bool isAllocate = false;
        bool isRecord = false;
        int entryOffset = 0; // bytes, inside the entry

        PTO_INTERNAL Producer() {}
        PTO_INTERNAL void setTileId(int t_id, int sub_t_id)
        {
            tile_id = t_id;
            sub_tile_id = sub_t_id;
        }
        PTO_INTERNAL int getTileId() const { return tile_id; }
        PTO_INTERNAL int getSubTileId() const { return sub_tile_id; }
        PTO_INTERNAL void setAllocateStatus(bool allocate) { isAllocate = allocate; }
        PTO_INTERNAL bool getAllocateStatus() const { return isAllocate; }
        PTO_INTERNAL void setRecordStatus(bool record) { isRecord = record; }
        PTO_INTERNAL bool getRecordStatus() const { return isRecord; }
        PTO_INTERNAL void setEntryOffset(int offset) { entryOffset = offset; }

        // wait until the consumer has released an entry
        PTO_INTERNAL void allocate() const { wait_flag_dev(FlagID + 1); }
        // the entry is filled
        PTO_INTERNAL void record() const
        {
            ffts_cross_core_sync(is_c2v ? PIPE_FIX : PIPE_MTE3, b200::ffts_config(FlagID));
        }
        PTO_INTERNAL void push(DataFiFo &fifo, TileDataProd &tile)
        {
            const uint32_t entry = static_cast<uint32_t>(tile_id) % static_cast<uint32_t>(DataFiFo::fifoDepth);
            T *addr = reinterpret_cast<T *>(reinterpret_cast<uint8_t *>(fifo.fifoBase) +
                                            static_cast<size_t>(entry) * kEntryElems * sizeof(T) + entryOffset);
            b200::entry_store<T, TileDataCons::Rows, TileDataCons::Cols>(addr, tile);
        }
    };

    struct Consumer {
        int tile_id = -1;
        int sub_tile_id = -1;
        bool isWait = false;
        bool isFree = false;
        int entryOffset = 0;

        PTO_INTERNAL Consumer() {}
        PTO_INTERNAL void setTileId(int tid, int sub_tid)
        {
            tile_id = tid;
            sub_tile_id = sub_tid;
        }
        PTO_INTERNAL int getTileId() const { return tile_id; }
        PTO_INTERNAL int getSubTileId() const { return sub_tile_id; }
        PTO_INTERNAL void setEntryOffset(int offset) { entryOffset = offset; }
        PTO_INTERNAL void setWaitStatus(bool wait) { isWait = wait; }
        PTO_INTERNAL bool getWaitStatus() const { return isWait; }
        PTO_INTERNAL void setFreeStatus(bool free) { isFree = free; }
        PTO_INTERNAL bool getFreeStatus() const { return isFree; }

        // wait until the producer has filled an entry
        PTO_INTERNAL void wait() const { wait_flag_dev(FlagID); }
        // the entry may be overwritten (the consumer's loads are complete)
        PTO_INTERNAL void free() const { ffts_cross_core_sync(PIPE_MTE2, b200::ffts_config(FlagID + 1)); }
        PTO_INTERNAL void pop(DataFiFo &fifo, TileDataCons &tile)
        {
            const uint32_t entry = static_cast<uint32_t>(tile_id) % static_cast<uint32_t>(DataFiFo::fifoDepth);
            T *addr = reinterpret_cast<T *>(reinterpret_cast<uint8_t *>(fifo.fifoBase) +
                                            static_cast<size_t>(entry) * kEntryElems * sizeof(T) + entryOffset);
            b200::entry_load<T, TileDataProd::Rows, TileDataProd::Cols>(addr, tile);
        }
    };

    DataFiFo fifo;
    Producer prod;
    Consumer cons;

    // `fifoBase`: the ring's storage, kEntryElems * FiFoDepth elements - global memory for a GM_FIFO, a tile's data()
    // in the block's arena for a VEC_FIFO / MAT_FIFO
    PTO_INTERNAL explicit TPipe(T *fifoBase) : fifo(fifoBase), prod(), cons() {}
};

// ---------------------------------------------------------------- TFIFOSync (the simulation's producer / consumer)
template <uint16_t FlagID, typename DataFIFOT, TSyncOpType ProducerOp, TSyncOpType ConsumerOp>
struct TFIFOSync {
    using Traits = TSyncTraits<ProducerOp, ConsumerOp>;
    static constexpr int fifoSize = DataFIFOT::fifoDepth;
    static constexpr int syncPeriod = DataFIFOT::fifoPeriod;

    struct Producer {
        int tile_id = 0;
        PTO_INTERNAL Producer() {}
        PTO_INTERNAL void set_tile_id(int t_id, int) { tile_id = t_id; }
        PTO_INTERNAL int get_tile_id() const { return tile_id; }
        PTO_INTERNAL void allocate() {}
        PTO_INTERNAL void record()
        {
            tile_id = (tile_id + 1) % fifoSize;
            ffts_cross_core_sync(Traits::is_cube_to_vec ? PIPE_FIX : PIPE_MTE3, b200::ffts_config(FlagID));
        }
    };
    struct Consumer {
        int tile_id = 0;
        int sub_tile_id = 0;
        PTO_INTERNAL Consumer() {}
        PTO_INTERNAL void set_tile_id(int tid, int) { tile_id = tid; }
        PTO_INTERNAL int get_tile_id() const { return tile_id; }
        PTO_INTERNAL void wait() { wait_flag_dev(FlagID); }
        PTO_INTERNAL void free() { tile_id = (tile_id + 1) % fifoSize; }
    };
};

namespace b200 {
template <typename P, typename = void>
struct is_pipe_endpoint : std::false_type {}; // TPipe's Producer / Consumer carry the status setters
template <typename P>
struct is_pipe_endpoint<P, std::void_t<decltype(std::declval<P &>().setEntryOffset(0))>> : std::true_type {};
} // namespace b200

// ---------------------------------------------------------------- TPUSH / TPOP / TFREE
// TPUSH: [allocate: wait for a free entry] -> store the tile into the entry -> [record: raise "entry filled"]
template <typename PipeProd, typename TileData, typename DataFifo, typename... WaitEvents>
PTO_INST RecordEvent TPUSH(PipeProd &prod, TileData &tile, DataFifo &fifo, WaitEvents &... events)
{
    TSYNC(events...);
    if constexpr (b200::is_pipe_endpoint<PipeProd>::value) {
        if (prod.getAllocateStatus()) {
            prod.allocate();
        }
        prod.push(fifo, tile);
        if (prod.getRecordStatus()) {
            prod.record();
        }
    } else {
        using T = typename DataFifo::DType;
        prod.allocate();
        T *addr = fifo.getBasePtr() + static_cast<size_t>(TileData::Numel) * (prod.get_tile_id() % DataFifo::fifoDepth);
        b200::entry_store<T, TileData::Rows, TileData::Cols>(addr, tile);
        prod.record();
    }
    return {};
}
template <typename TileData, typename Pipe, typename... WaitEvents,
          std::enable_if_t<is_tile<TileData>::value, int> = 0>
PTO_INST RecordEvent TPUSH(TileData &tile, Pipe &pipe, WaitEvents &... events)
{
    return TPUSH(pipe.prod, tile, pipe.fifo, events...);
}

// TPOP: [wait for a filled entry] -> load the entry into the tile -> [free: raise "entry free again"]
template <typename PipeCons, typename TileData, typename DataFifo, typename... WaitEvents>
PTO_INST RecordEvent TPOP(PipeCons &cons, TileData &tile, DataFifo &fifo, WaitEvents &... events)
{
    TSYNC(events...);
    if constexpr (b200::is_pipe_endpoint<PipeCons>::value) {
        if (cons.getWaitStatus()) {
            cons.wait();
        }
        cons.pop(fifo, tile);
        if (cons.getFreeStatus()) {
            cons.free();
        }
    } else {
        using T = typename DataFifo::DType;
        cons.wait();
        T *addr = fifo.getBasePtr() + static_cast<size_t>(TileData::Numel) * (cons.get_tile_id() % DataFifo::fifoDepth);
        b200::entry_load<T, TileData::Rows, TileData::Cols>(addr, tile);
        cons.free();
    }
    return {};
}
template <typename TileData, typename Pipe, typename... WaitEvents,
          std::enable_if_t<is_tile<TileData>::value, int> = 0>
PTO_INST RecordEvent TPOP(TileData &tile, Pipe &pipe, WaitEvents &... events)
{
    return TPOP(pipe.cons, tile, pipe.fifo, events...);
}

// TFREE: release the entry last popped, when the consumer was told to
template <typename Pipe, typename... WaitEvents>
PTO_INST RecordEvent TFREE(Pipe &pipe, WaitEvents &... events)
{
    TSYNC(events...);
    if (pipe.cons.getFreeStatus()) {
        pipe.cons.free();
    }
    return {};
}

} // namespace pto
