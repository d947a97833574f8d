#pragma once
#include "common.cuh"
#include "ctx.h"
namespace p0p {
inline bool umma_supported(const p0p_ctx*, const KP&) { return false; }
inline int launch_umma(p0p_ctx*, const KP&) { return -9; }
}
