// Tile programs of the reference include this path directly; everything lives in the backend headers.
#pragma once
#include "../pto-inst.hpp"
