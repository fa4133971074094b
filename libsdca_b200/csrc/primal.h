// W = [W0 +] X A' on the current device: the primal variables of a feature
// problem rebuilt from the dual ones (eval_recompute_primal of the reference,
// include/sdca/solver/eval/core.h:148-182).
#pragma once

#include <cuda_runtime.h>

namespace sdcab {

// x: d x n column major, a: m x n column major, w0 (optional) and w: d x m column
// major.  The sum over the examples runs in increasing order within a slice of
// examples and over the slices in increasing order: the result does not depend
// on the launch.
template <typename Data>
int primal_from_dual_dev(const Data* x, const Data* a, const Data* w0, Data* w, long long d,
                         long long m, long long n, cudaStream_t stream);

// test switch: 1 keeps float data on the CUDA-core kernel
void primal_test_force_simt(int on);

}  // namespace sdcab
