// Register-resident fast paths for the common shapes (placeholder dispatch).
#pragma once
#include "common_host.h"
#include "prox_core.cuh"
namespace sdcab {
constexpr int kNoFastPath = 1;
template <typename Data, typename R>
int launch_fast_rows(int, const Data*, Data*, int, long long, const ProxParams&, cudaStream_t) { return kNoFastPath; }
}
