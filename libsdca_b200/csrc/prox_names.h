// Operator names accepted by the C ABI: the strings matsdca_prox dispatches on
// (src/matlab/mex_prox.cpp:143-176 of the reference).
#pragma once

#include <cstring>

#include "prox_core.cuh"

namespace sdcab {

inline int prox_id_from_name(const char* name) {
  if (!name) return -1;
  struct Entry { const char* name; int id; };
  static const Entry table[] = {
      {"knapsack", kKnapsackEq},
      {"knapsack_eq", kKnapsackEq},
      {"knapsack_le", kKnapsackLe},
      {"knapsack_le_biased", kKnapsackLeBiased},
      {"topk_simplex", kTopkSimplex},
      {"topk_simplex_biased", kTopkSimplexBiased},
      {"topk_cone", kTopkCone},
      {"topk_cone_biased", kTopkConeBiased},
      {"entropy", kEntropy},
      {"entropy_norm", kEntropyNorm},
      {"topk_entropy", kTopkEntropy},
      {"topk_entropy_biased", kTopkEntropyBiased},
      {"two_simplex", kTwoSimplex},
      // the sort-based variant is its own routine (two_simplex_sort.cuh): it differs
      // from two_simplex where a block ends up empty or the common sum is zero
      {"two_simplex_sort", kTwoSimplexSort},
      {"lambert_w_exp", kLambertWExp},
  };
  for (const Entry& e : table)
    if (std::strcmp(e.name, name) == 0) return e.id;
  return -1;
}

}  // namespace sdcab
