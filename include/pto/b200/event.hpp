// Typed events of the PTO surface: Event<SrcOp, DstOp> names the dependency "everything of kind SrcOp issued so far
// must be complete before the next DstOp starts" and is carried by the flag of the two operations' pipes
// (include/pto/common/event.hpp:19-154 and include/pto/npu/a2a3/TSync.hpp:25-228 in the reference: `Op`, the
// operation -> pipe table, Event::Init / Record / Wait, `event = TXXX(...)`, and TXXX(..., events...) which waits
// for its events first).  On this backend a flag is an mbarrier of the block (runtime.hpp); an automatic event id is
// taken in turn from the pair's eight ids.
#pragma once

#include "runtime.hpp"

namespace pto {

enum class Op : uint16_t {
    TLOAD, TSTORE_VEC, SCALAR, TRESHAPE, VECTOR, TADD, TADDS, TSUB, TMUL, TMULS, TDIV, TDIVS, TMIN, TMINS, TMAX, TAND,
    TOR, TSEL, TSHL, TSHR, TEXP, TSELS, TSQRT, TRSQRT, TEXPANDS, TPARTADD, TPARTMUL, TPARTMAX, TPARTMIN, TCMPS,
    TMRGSORT, TSORT32, TCI, TGATHER, TGATHERB, TCVT, TROWSUM, TROWPROD, TROWMAX, TROWMIN, TROWEXPAND, TCOLSUM,
    TCOLPROD, TCOLMAX, TCOLMIN, TTRANS, TTRI, TREM, TFMOD, TREMS, TFMODS, TSUBS, TMAXS, TLRELU, TPRELU, TMOV_V2V,
    TMOV_V2M, TEXTRACT_V2M, TMOV_M2B, TMOV_M2L, TMOV_M2R, TMOV_M2S, TMOV_A2V, TMOV_A2M, TSTORE_ACC, TSTORE_MAT,
    TMATMUL, TGEMV, TMATMUL_MX, TEXTRACT_M2LR, TANDS, TORS, TSHLS, TSHRS, TXOR, TXORS, TEXTRACT_A2M, TINSERT_A2M,
    TIMG2COL, TSETFMATRIX, TSET_IMG2COL_RPT, TSET_IMG2COL_PADDING, TDEQUANT,
    OP_COUNT,
};

namespace b200 {
// the pipe an operation runs on (the reference's opPipeList, include/pto/npu/a2a3/TSync.hpp:26-110)
constexpr pipe_t pipe_of(Op op)
{
    switch (op) {
        case Op::TLOAD: return PIPE_MTE2;
        case Op::TSTORE_VEC:
        case Op::TSTORE_MAT: return PIPE_MTE3;
        case Op::SCALAR:
        case Op::TRESHAPE:
        case Op::TCI:
        case Op::TSETFMATRIX:
        case Op::TSET_IMG2COL_RPT:
        case Op::TSET_IMG2COL_PADDING: return PIPE_S;
        case Op::TMOV_V2M:
        case Op::TEXTRACT_V2M:
        case Op::TMOV_M2S:
        case Op::TMOV_A2V:
        case Op::TMOV_A2M:
        case Op::TSTORE_ACC:
        case Op::TEXTRACT_A2M:
        case Op::TINSERT_A2M: return PIPE_FIX;
        case Op::TMOV_M2B:
        case Op::TMOV_M2L:
        case Op::TMOV_M2R:
        case Op::TEXTRACT_M2LR:
        case Op::TIMG2COL: return PIPE_MTE1;
        case Op::TMATMUL:
        case Op::TGEMV:
        case Op::TMATMUL_MX: return PIPE_M;
        case Op::OP_COUNT: return PIPE_ALL;
        default: return PIPE_V;
    }
}
} // namespace b200

template <Op OpCode>
PTO_INTERNAL constexpr pipe_t GetPipeByOp()
{
    return b200::pipe_of(OpCode);
}

template <Op SrcOp, Op DstOp, bool AutoToken = true, event_t EventID = EVENT_ID0>
struct Event {
    static constexpr Op srcOp = SrcOp;
    static constexpr Op dstOp = DstOp;
    static constexpr pipe_t srcPipe = b200::pipe_of(SrcOp);
    static constexpr pipe_t dstPipe = b200::pipe_of(DstOp);
    static_assert(SrcOp != DstOp, "SrcOp is not allowed to be equal to DstOp.");
    static_assert(srcPipe != dstPipe, "SrcPipe is not allowed to be equal to dstPipe.");

    // an accumulator leaving the cube role for the vector role, or a vector tile entering the cube role's L1
    static constexpr bool IsCrossCore = ((SrcOp == Op::TMOV_A2V) && (dstPipe == PIPE_V)) ||
                                        ((SrcOp == Op::TMOV_V2M || SrcOp == Op::TEXTRACT_V2M) && (dstPipe == PIPE_MTE1));
    static_assert(!IsCrossCore || !AutoToken, "Cross-core events must manually specify EventID.");

    const event_t token = AutoToken ? b200::next_event_id(srcPipe, dstPipe) : EventID;

    PTO_INTERNAL Event() {}

    PTO_INTERNAL Event &InitAddr(uint64_t)
    {
        static_assert(IsCrossCore, "Only cross-core events require setting the initial addr.");
        return *this;
    }

    template <uint8_t CrossCoreId = 0xff>
    PTO_INTERNAL Event &Wait()
    {
        if constexpr (IsCrossCore) {
            static_assert(CrossCoreId != 0xff, "The cross-core id must be assigned when the event is a cross-core event.");
            wait_flag_dev(CrossCoreId);
        } else {
            wait_flag(srcPipe, dstPipe, token);
        }
        return *this;
    }

    template <uint8_t CrossCoreId = 0xff>
    PTO_INTERNAL Event &Init()
    {
        if constexpr (IsCrossCore) {
            static_assert(CrossCoreId != 0xff, "The cross-core id must be assigned when the event is a cross-core event.");
            ffts_cross_core_sync(srcPipe, (static_cast<uint64_t>(CrossCoreId) & 0xf) << 8 | 0x21u);
        } else {
            set_flag(srcPipe, dstPipe, token);
        }
        return *this;
    }

    template <uint8_t CrossCoreId = 0xff>
    PTO_INTERNAL Event &Record()
    {
        return Init<CrossCoreId>();
    }

    // `event = TXXX(...)`: the instruction just issued is the one the event records
    PTO_INTERNAL Event &operator=(RecordEvent)
    {
        static_assert(!IsCrossCore, "A cross-core event must be initialised with its cross-core id.");
        return Init();
    }
};

template <typename... WaitEvents>
PTO_INTERNAL void WaitAllEvents(WaitEvents &... events)
{
    (events.Wait(), ...);
}

// TSYNC(events...): wait for every event; TSYNC<Op>(): a barrier on the (vector) pipe of Op
template <typename... WaitEvents>
PTO_INST void TSYNC(WaitEvents &... events)
{
    WaitAllEvents(events...);
}
template <Op OpCode>
PTO_INST void TSYNC()
{
    static_assert(b200::pipe_of(OpCode) == PIPE_V, "Single Op TSYNC only supports Vector PTO Instruction.");
    pipe_barrier(PIPE_V);
}

template <pipe_t SrcPipe, pipe_t DstPipe>
PTO_INTERNAL void PtoSetWaitFlag()
{
    set_flag(SrcPipe, DstPipe, EVENT_ID0);
    wait_flag(SrcPipe, DstPipe, EVENT_ID0);
}

} // namespace pto
