// Geometry of the attention kernels: feature width K = 2 * proj_dim = 128, head dim d = 64.
#pragma once

#include "common.cuh"

namespace rfa {

constexpr int kK = 128;        // width of phi
constexpr int kD = 64;         // head dim

}  // namespace rfa
