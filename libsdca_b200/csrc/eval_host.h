// Host-side pieces of the evaluation: objective names and the step from summed
// per-example terms to the evaluation record.
#pragma once

#include <cmath>
#include <cstring>
#include <limits>

#include "../../include/sdca_b200.h"
#include "losses.cuh"

namespace sdcab {

// Objective names and parameter rules of matsdca_fit
// (src/matlab/mex_solve.cpp:622-719 of the reference).
inline int objective_from_name(const char* name, double c, double gamma, int64_t k,
                               sdcab_objective* out) {
  if (!name || !out) return SDCAB_ERR_ARG;
  if (!(c > 0) || !(gamma >= 0) || k < 1) return SDCAB_ERR_ARG_RANGE;
  auto is = [&](const char* a, const char* b = nullptr) {
    return std::strcmp(name, a) == 0 || (b && std::strcmp(name, b) == 0);
  };
  int id = -1;
  if (is("msvm", "l2_multiclass_hinge")) {
    if (k != 1) return SDCAB_ERR_ARG_RANGE;
    id = SDCAB_OBJ_L2_TOPK_HINGE;
  } else if (is("msvm_smooth", "l2_multiclass_hinge_smooth")) {
    if (k != 1) return SDCAB_ERR_ARG_RANGE;
    id = SDCAB_OBJ_L2_TOPK_HINGE_SMOOTH;
  } else if (is("softmax", "l2_multiclass_entropy")) {
    if (k != 1) return SDCAB_ERR_ARG_RANGE;
    id = SDCAB_OBJ_L2_ENTROPY;
  } else if (is("l2_hinge_topk", "topk_hinge_alpha")) {
    id = gamma > 0 ? SDCAB_OBJ_L2_HINGE_TOPK_SMOOTH : SDCAB_OBJ_L2_HINGE_TOPK;
  } else if (is("l2_topk_hinge", "topk_hinge_beta")) {
    id = gamma > 0 ? SDCAB_OBJ_L2_TOPK_HINGE_SMOOTH : SDCAB_OBJ_L2_TOPK_HINGE;
  } else if (is("l2_entropy_topk")) {
    id = SDCAB_OBJ_L2_ENTROPY_TOPK;
  } else if (is("mlsvm", "l2_multilabel_hinge")) {
    id = SDCAB_OBJ_L2_MULTILABEL_HINGE;
  } else if (is("mlsvm_smooth", "l2_multilabel_hinge_smooth")) {
    id = SDCAB_OBJ_L2_MULTILABEL_HINGE_SMOOTH;
  } else if (is("mlsoftmax", "l2_multilabel_entropy")) {
    id = SDCAB_OBJ_L2_MULTILABEL_ENTROPY;
  } else {
    return SDCAB_ERR_OBJECTIVE;
  }
  const bool smooth = (id == SDCAB_OBJ_L2_HINGE_TOPK_SMOOTH || id == SDCAB_OBJ_L2_TOPK_HINGE_SMOOTH ||
                       id == SDCAB_OBJ_L2_MULTILABEL_HINGE_SMOOTH);
  if (smooth && !(gamma > 0)) return SDCAB_ERR_ARG_RANGE;
  out->id = id; out->precision = SDCAB_PRECISION_DOUBLE;
  out->c = c; out->gamma = gamma; out->k = k;
  return SDCAB_OK;
}

inline int check_objective(const sdcab_objective* o, int64_t m) {
  if (!o) return SDCAB_ERR_ARG;
  if (o->id < 0 || o->id >= kNumObjectives) return SDCAB_ERR_OBJECTIVE;
  if (!(o->c > 0) || !(o->gamma >= 0)) return SDCAB_ERR_ARG_RANGE;
  const bool has_k = (o->id >= SDCAB_OBJ_L2_ENTROPY_TOPK && o->id <= SDCAB_OBJ_L2_TOPK_HINGE_SMOOTH);
  if (has_k && (o->k < 1 || o->k > m - 1)) return SDCAB_ERR_ARG_RANGE;  // mex_solve.cpp:641
  if (o->precision != SDCAB_PRECISION_DOUBLE && o->precision != SDCAB_PRECISION_FLOAT)
    return SDCAB_ERR_PRECISION;
  return SDCAB_OK;
}

// The label checks of the reference (include/sdca/solver/data/output.h:169-215)
// on host arrays, labels 0-based: every label inside [0, m); multilabel examples
// have offsets[0] == 0, between 1 and m - 1 labels each, and their labels
// strictly increasing (distinct and sorted).
inline int validate_labels(const int64_t* labels, const int64_t* offsets, int64_t n, int64_t m,
                           bool multilabel) {
  if (!labels || n < 0) return SDCAB_ERR_ARG;
  if (!multilabel) {
    for (int64_t i = 0; i < n; ++i)
      if (labels[i] < 0 || labels[i] >= m) return SDCAB_ERR_LABELS_RANGE;
    return SDCAB_OK;
  }
  if (!offsets) return SDCAB_ERR_ARG;
  if (offsets[0] != 0) return SDCAB_ERR_LABELS_RANGE;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t first = offsets[i], count = offsets[i + 1] - first;
    if (count < 1 || count >= m) return SDCAB_ERR_LABELS_RANGE;
    for (int64_t q = 0; q < count; ++q) {
      const int64_t c = labels[first + q];
      if (c < 0 || c >= m) return SDCAB_ERR_LABELS_RANGE;
      if (q > 0 && c <= labels[first + q - 1]) return SDCAB_ERR_LABELS_RANGE;
    }
  }
  return SDCAB_OK;
}

inline ObjectiveParams to_params(const sdcab_objective* o) {
  ObjectiveParams q;
  q.id = o->id; q.k = static_cast<int>(o->k); q.c = o->c; q.gamma = o->gamma;
  return q;
}

// eval_end (include/sdca/solver/eval/core.h:43-132) and update_all
// (objective/objective_base.h:108-128) on the summed terms.
inline int eval_finish(const sdcab_objective* obj, int64_t m, const double* sums,
                       sdcab_eval_record* rec, double* accuracy) {
  if (!obj || !sums || !rec || m < 1) return SDCAB_ERR_ARG;
  if (sums[6] != 0.0) return SDCAB_ERR_TIMEOUT;  // a bounded device wait ran out
  const ObjectiveParams q = to_params(obj);
  const double n = sums[5];
  rec->primal_loss = sums[0] * objective_coeff(q);
  rec->dual_loss = sums[1];
  rec->primal_regularizer = sums[2];
  rec->dual_regularizer = sums[3];
  rec->primal = rec->primal_loss + rec->primal_regularizer;
  rec->dual = rec->dual_loss - rec->dual_regularizer;
  rec->rank_loss = (n > 0) ? sums[4] / n : 0.0;
  // eval/types.h:34-41
  const double mx = std::fmax(std::fabs(rec->primal), std::fabs(rec->dual));
  rec->relative_gap = (mx > 0) ? (mx < std::numeric_limits<double>::infinity()
                                      ? (rec->primal - rec->dual) / mx
                                      : std::numeric_limits<double>::infinity())
                               : 0.0;
  if (accuracy) {
    double run = 0;
    const double coeff = (n > 0) ? 1.0 / n : 0.0;
    for (int64_t j = 0; j < m; ++j) {
      run += sums[8 + j];
      accuracy[j] = run * coeff;
    }
  }
  return SDCAB_OK;
}

}  // namespace sdcab
