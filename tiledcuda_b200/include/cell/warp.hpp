// Warp shuffles (reference: include/cell/warp.hpp:13-26).
#pragma once

#include "config.hpp"

namespace tiledcuda::cell {

template <typename T>
DEVICE T shuffle_sync(T value, int src_lane) {
    return __shfl_sync(0xffffffffu, value, src_lane);
}

template <typename T>
DEVICE T shuffle_down_sync(T value, int delta) {
    return __shfl_down_sync(0xffffffffu, value, delta);
}

template <typename T>
DEVICE T shuffle_xor_sync(T value, int lane_mask) {
    return __shfl_xor_sync(0xffffffffu, value, lane_mask);
}

}  // namespace tiledcuda::cell
