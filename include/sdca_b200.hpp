// Header-only C++ shim over the C ABI with the reference's function names and
// argument order, so that callers written against libsdca's headers switch by
// namespace:  sdca::prox_topk_simplex(dim, first, last, aux, k, rhs)  becomes
// sdca::b200::prox_topk_simplex(dim, first, last, aux, k, rhs).
//
// Pointers are host pointers (the batched overloads of include/sdca/prox/*.h
// and evaluate_dataset of include/sdca/solver/eval.h work on host memory); the
// data goes to the current CUDA device and back inside the call.  `aux` is
// accepted for signature compatibility and not used (the device kernels need
// no per-row scratch).  Errors are reported the way the reference's front end
// reports them: a std::runtime_error carrying the LIBSDCA:* identifier.
#ifndef SDCA_B200_HPP
#define SDCA_B200_HPP

#include <cstddef>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "sdca_b200.h"

namespace sdca {
namespace b200 {

inline void check(int status, const char* what) {
  if (status != SDCAB_OK) {
    throw std::runtime_error(std::string(what) + ": " + sdcab_status_string(status) + " " +
                             sdcab_last_error());
  }
}

template <typename Result> struct precision_of;
template <> struct precision_of<double> { static const int value = SDCAB_PRECISION_DOUBLE; };
template <> struct precision_of<float> { static const int value = SDCAB_PRECISION_FLOAT; };

namespace detail {
inline int call(const char* name, float* a, std::ptrdiff_t m, std::ptrdiff_t n, const sdcab_prox_opts& o) {
  return sdcab_prox_f32(name, a, m, n, &o, nullptr);
}
inline int call(const char* name, double* a, std::ptrdiff_t m, std::ptrdiff_t n, const sdcab_prox_opts& o) {
  return sdcab_prox_f64(name, a, m, n, &o, nullptr);
}
template <typename Result, typename Data>
inline void run(const char* name, std::ptrdiff_t dim, Data* first, Data* last, sdcab_prox_opts o) {
  o.precision = precision_of<Result>::value;
  check(call(name, first, dim, (last - first) / dim, o), name);
}
inline sdcab_prox_opts defaults() {
  sdcab_prox_opts o;
  sdcab_prox_opts_default(&o);
  return o;
}
}  // namespace detail

// include/sdca/prox/knapsack_eq.h:143-157
template <typename Result = double, typename Data>
inline void prox_knapsack_eq(std::ptrdiff_t dim, Data* first, Data* last, Data* /*aux*/,
                             Result lo = 0, Result hi = 1, Result rhs = 1) {
  sdcab_prox_opts o = detail::defaults(); o.lo = lo; o.hi = hi; o.rhs = rhs;
  detail::run<Result>("knapsack_eq", dim, first, last, o);
}
// include/sdca/prox/knapsack_le.h:78-92
template <typename Result = double, typename Data>
inline void prox_knapsack_le(std::ptrdiff_t dim, Data* first, Data* last, Data*,
                             Result lo = 0, Result hi = 1, Result rhs = 1) {
  sdcab_prox_opts o = detail::defaults(); o.lo = lo; o.hi = hi; o.rhs = rhs;
  detail::run<Result>("knapsack_le", dim, first, last, o);
}
// include/sdca/prox/knapsack_le_biased.h:165-180
template <typename Result = double, typename Data>
inline void prox_knapsack_le_biased(std::ptrdiff_t dim, Data* first, Data* last, Data*,
                                    Result lo = 0, Result hi = 1, Result rhs = 1, Result rho = 1) {
  sdcab_prox_opts o = detail::defaults(); o.lo = lo; o.hi = hi; o.rhs = rhs; o.rho = rho;
  detail::run<Result>("knapsack_le_biased", dim, first, last, o);
}
// include/sdca/prox/topk_simplex.h:100-113
template <typename Result = double, typename Data>
inline void prox_topk_simplex(std::ptrdiff_t dim, Data* first, Data* last, Data*,
                              std::ptrdiff_t k = 1, Result rhs = 1) {
  sdcab_prox_opts o = detail::defaults(); o.k = k; o.rhs = rhs;
  detail::run<Result>("topk_simplex", dim, first, last, o);
}
// include/sdca/prox/topk_simplex_biased.h:105-119
template <typename Result = double, typename Data>
inline void prox_topk_simplex_biased(std::ptrdiff_t dim, Data* first, Data* last, Data*,
                                     std::ptrdiff_t k = 1, Result rhs = 1, Result rho = 1) {
  sdcab_prox_opts o = detail::defaults(); o.k = k; o.rhs = rhs; o.rho = rho;
  detail::run<Result>("topk_simplex_biased", dim, first, last, o);
}
// include/sdca/prox/topk_cone.h:187-199
template <typename Result = double, typename Data>
inline void prox_topk_cone(std::ptrdiff_t dim, Data* first, Data* last, Data*, std::ptrdiff_t k = 1) {
  sdcab_prox_opts o = detail::defaults(); o.k = k;
  detail::run<Result>("topk_cone", dim, first, last, o);
}
// include/sdca/prox/topk_cone_biased.h:145-158
template <typename Result = double, typename Data>
inline void prox_topk_cone_biased(std::ptrdiff_t dim, Data* first, Data* last, Data*,
                                  std::ptrdiff_t k = 1, Result rho = 1) {
  sdcab_prox_opts o = detail::defaults(); o.k = k; o.rho = rho;
  detail::run<Result>("topk_cone_biased", dim, first, last, o);
}
// include/sdca/prox/entropy.h:85-98
template <typename Result = double, typename Data>
inline void prox_entropy(std::ptrdiff_t dim, Data* first, Data* last, Data*, Result hi = 1, Result rhs = 1) {
  sdcab_prox_opts o = detail::defaults(); o.hi = hi; o.rhs = rhs;
  detail::run<Result>("entropy", dim, first, last, o);
}
// include/sdca/prox/entropy_norm.h:213-226
template <typename Result = double, typename Data>
inline void prox_entropy_norm(std::ptrdiff_t dim, Data* first, Data* last, Data*, Result hi = 1, Result rhs = 1) {
  sdcab_prox_opts o = detail::defaults(); o.hi = hi; o.rhs = rhs;
  detail::run<Result>("entropy_norm", dim, first, last, o);
}
// include/sdca/prox/topk_entropy.h:106-118
template <typename Result = double, typename Data>
inline void prox_topk_entropy(std::ptrdiff_t dim, Data* first, Data* last, Data*, std::ptrdiff_t k = 1) {
  sdcab_prox_opts o = detail::defaults(); o.k = k;
  detail::run<Result>("topk_entropy", dim, first, last, o);
}
// include/sdca/prox/topk_entropy_biased.h:302-315
template <typename Result = double, typename Data>
inline void prox_topk_entropy_biased(std::ptrdiff_t dim, Data* first, Data* last, Data*,
                                     std::ptrdiff_t k = 1, Result alpha = 1) {
  sdcab_prox_opts o = detail::defaults(); o.k = k; o.alpha = alpha;
  detail::run<Result>("topk_entropy_biased", dim, first, last, o);
}
// include/sdca/prox/two_simplex.h:183-196 (dim, p, first, last, aux, rhs)
template <typename Result = double, typename Data>
inline void prox_two_simplex(std::ptrdiff_t dim, std::ptrdiff_t p, Data* first, Data* last, Data*,
                             Result rhs = 1) {
  sdcab_prox_opts o = detail::defaults(); o.p = p; o.rhs = rhs;
  detail::run<Result>("two_simplex", dim, first, last, o);
}
// include/sdca/prox/two_simplex_sort.h:177-189 (dim, p, first, last, aux, rhs): the sort-based
// routine, a different function from two_simplex where a block ends up empty
template <typename Result = double, typename Data>
inline void prox_two_simplex_sort(std::ptrdiff_t dim, std::ptrdiff_t p, Data* first, Data* last, Data*,
                                  Result rhs = 1) {
  sdcab_prox_opts o = detail::defaults(); o.p = p; o.rhs = rhs;
  detail::run<Result>("two_simplex_sort", dim, first, last, o);
}
// apply(dim, first, last, lambert_w_exp_map<Data>()): include/sdca/prox/proxdef.h:386-400
template <typename Data>
inline void apply_lambert_w_exp(std::ptrdiff_t dim, Data* first, Data* last) {
  detail::run<double>("lambert_w_exp", dim, first, last, detail::defaults());
}

// evaluate_dataset (include/sdca/solver/eval.h:15-51) on host buffers: the
// objective by its matsdca_fit name, the problem in the reference's memory
// layout; returns the record and fills `accuracy` (m entries) if not empty.
template <typename Data>
inline sdcab_eval_record evaluate_dataset(const sdcab_objective& objective, const sdcab_problem& problem,
                                          std::vector<double>* accuracy = nullptr) {
  sdcab_eval_record rec;
  double* acc = nullptr;
  if (accuracy) { accuracy->assign(static_cast<std::size_t>(problem.m), 0.0); acc = accuracy->data(); }
  if (std::is_same<Data, float>::value) check(sdcab_eval_f32(&objective, &problem, &rec, acc), "evaluate_dataset");
  else check(sdcab_eval_f64(&objective, &problem, &rec, acc), "evaluate_dataset");
  return rec;
}

// solver::solve (include/sdca/solver.h:39-52) on host buffers: runs epochs of
// SDCA steps until the reference's stopping rule ends them; `problem.a` (and
// `problem.w` for features) hold the starting point and receive the result.
// Returns status / epoch count; `evals` receives one record per evaluation.
template <typename Data>
inline sdcab_fit_result solve(const sdcab_objective& objective, const sdcab_problem& problem,
                              const sdcab_fit_criteria& criteria,
                              std::vector<sdcab_eval_record>* evals = nullptr) {
  sdcab_fit_result res;
  std::vector<sdcab_eval_record> local(static_cast<std::size_t>(criteria.max_epoch) + 4);
  const int rc = std::is_same<Data, float>::value
      ? sdcab_fit_f32(&objective, &problem, &criteria, nullptr, local.data(),
                      static_cast<int64_t>(local.size()), &res)
      : sdcab_fit_f64(&objective, &problem, &criteria, nullptr, local.data(),
                      static_cast<int64_t>(local.size()), &res);
  check(rc, "solve");
  if (evals) evals->assign(local.begin(), local.begin() + static_cast<std::ptrdiff_t>(res.num_evals));
  return res;
}

}  // namespace b200
}  // namespace sdca

#endif  // SDCA_B200_HPP
