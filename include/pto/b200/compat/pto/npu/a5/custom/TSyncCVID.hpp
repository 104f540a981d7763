// Same interface as the a2a3 header of this name (the reference keeps one per NPU generation).
#pragma once
#include "../../a2a3/custom/TSyncCVID.hpp"
