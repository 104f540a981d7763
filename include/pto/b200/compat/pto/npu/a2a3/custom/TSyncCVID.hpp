// TSYNC_CVID of the reference (include/pto/npu/a2a3/custom/TSyncCVID.hpp:33-85): on the NPU the cube core of a block
// tells its vector cores which communication slot (a physical core number modulo the slot count) the block's FIFOs use.
// Here one thread block plays the cube and the vector role of a logical block, so the slot is the block index itself,
// taken modulo the slot count like the reference's.  The message helper builds the same word that
// ffts_cross_core_sync reads the flag id from (bits 8..11).
#pragma once
#include <cstdint>

namespace pto {

enum CVCommFlag : uint32_t { CV_COMM_CTRL = 12, CV_COMM_RSVD_13, CV_COMM_RSVD_14, CV_COMM_RSVD_15 };

constexpr int kCvCommSlotBytes = 512;
constexpr int kCvMaxCores = 25;

enum CVSyncMode : uint16_t { C_ALL_CORE_SYNC = 0, V_ALL_CORE_SYNC = 0, V_SUBCORES_SYNC = 1, CV_CORE_SYNC = 2 };

AICORE inline uint16_t _getFFTSMsg(CVSyncMode mode, uint16_t flag_id, uint16_t base_const = 0x1)
{
    return static_cast<uint16_t>((base_const & 0xf) | ((mode & 0x3) << 4) | ((flag_id & 0xf) << 8));
}

template <int CV_COMM_SLOT_BYTES = kCvCommSlotBytes, int CV_MAX_CORES = kCvMaxCores>
AICORE inline int TSYNC_CVID(int block_idx, __gm__ uint8_t *cv_comm_buf)
{
    (void)cv_comm_buf;
    return block_idx % CV_MAX_CORES;
}

} // namespace pto
