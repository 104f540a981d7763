// Include-path compatibility: the reference's kernels include <pto/common/debug.hpp>; on this backend everything comes
// with the entry header.
#pragma once
#include <pto/pto-inst.hpp>
