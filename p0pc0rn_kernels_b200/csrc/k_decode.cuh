#pragma once
#include "common.cuh"
#include "ctx.h"
namespace p0p {
inline bool decode_supported(const KP&) { return false; }
inline int launch_decode(p0p_ctx*, const KP&) { return -9; }
}
