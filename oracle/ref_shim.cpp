/*
 * Test infrastructure: C entry points over the UNMODIFIED reference headers.
 *
 * This file is compiled against the reference's own include/ tree (the path is
 * given on the compiler command line by oracle/build_oracle.py; nothing of the
 * reference is copied here) into oracle/_ref/libsdca_ref.so.  It instantiates
 * the reference templates for float/double data and float/double result
 * precision and exposes them with plain-C signatures so that tests can compare
 * the CUDA library and the C restatement in oracle/sdca_oracle.c against the
 * reference itself, and so that bench.py can time the reference's CPU path.
 *
 * Reference entry points wrapped here (paths inside the reference project):
 *   include/sdca/prox/\*.h       batched prox_<name>(dim, first, last, aux, ...)
 *                                 and thresholds_<name>(first, last, ...)
 *   include/sdca/prox/proxdef.h   apply(dim, first, last, functor)   (:386-400)
 *   include/sdca/solver/eval.h    evaluate_dataset                   (:15-51)
 *   include/sdca/solver.h         solver::solve                      (:39-51)
 *
 * Only tests, the smoke check and bench.py's CPU-baseline leg may load the
 * library built from this file.
 */
#include <cstdint>
#include <cstring>
#include <functional>
#include <limits>
#include <string>
#include <thread>
#include <vector>

#include "sdca/prox.h"
#include "sdca/solver.h"
#include "sdca/utility/logging.cpp"

namespace {

struct ref_opts {
  double lo, hi, rhs, rho, alpha;
  int64_t k, p;
};

typedef std::ptrdiff_t idx_t;

// ---------------------------------------------------------------- prox -----
template <typename Data, typename Result>
int run_prox(const std::string& name, Data* first, idx_t m, idx_t n,
             const ref_opts& o) {
  using namespace sdca;
  std::vector<Data> aux_vec(static_cast<std::size_t>(m));
  Data* aux = aux_vec.data();
  Data* last = first + m * n;
  Result lo = static_cast<Result>(o.lo), hi = static_cast<Result>(o.hi);
  Result rhs = static_cast<Result>(o.rhs), rho = static_cast<Result>(o.rho);
  Result alpha = static_cast<Result>(o.alpha);
  idx_t k = static_cast<idx_t>(o.k), p = static_cast<idx_t>(o.p);
  if (name == "knapsack" || name == "knapsack_eq") {
    prox_knapsack_eq(m, first, last, aux, lo, hi, rhs);
  } else if (name == "knapsack_le") {
    prox_knapsack_le(m, first, last, aux, lo, hi, rhs);
  } else if (name == "knapsack_le_biased") {
    prox_knapsack_le_biased(m, first, last, aux, lo, hi, rhs, rho);
  } else if (name == "topk_simplex") {
    prox_topk_simplex(m, first, last, aux, k, rhs);
  } else if (name == "topk_simplex_biased") {
    prox_topk_simplex_biased(m, first, last, aux, k, rhs, rho);
  } else if (name == "two_simplex") {
    prox_two_simplex(m, p, first, last, aux, rhs);
  } else if (name == "two_simplex_sort") {
    prox_two_simplex_sort(m, p, first, last, aux, rhs);
  } else if (name == "topk_entropy") {
    prox_topk_entropy<Result>(m, first, last, aux, k);
  } else if (name == "topk_entropy_biased") {
    prox_topk_entropy_biased(m, first, last, aux, k, alpha);
  } else if (name == "entropy") {
    prox_entropy(m, first, last, aux, hi, rhs);
  } else if (name == "entropy_norm") {
    prox_entropy_norm(m, first, last, aux, hi, rhs);
  } else if (name == "topk_cone") {
    prox_topk_cone<Result>(m, first, last, aux, k);
  } else if (name == "topk_cone_biased") {
    prox_topk_cone_biased(m, first, last, aux, k, rho);
  } else if (name == "lambert_w_exp") {
    apply(m, first, last, lambert_w_exp_map<Data>());
  } else {
    return -1;
  }
  return 0;
}

template <typename Data, typename Result>
int run_prox_threads(const std::string& name, Data* a, idx_t m, idx_t n,
                     const ref_opts& o, int nthreads) {
  if (nthreads <= 1 || n < 2 * nthreads) {
    return run_prox<Data, Result>(name, a, m, n, o);
  }
  std::vector<std::thread> pool;
  std::vector<int> rc(static_cast<std::size_t>(nthreads), 0);
  for (int t = 0; t < nthreads; ++t) {
    idx_t r0 = n * t / nthreads, r1 = n * (t + 1) / nthreads;
    pool.emplace_back([&, t, r0, r1]() {
      rc[static_cast<std::size_t>(t)] =
          run_prox<Data, Result>(name, a + m * r0, m, r1 - r0, o);
    });
  }
  for (auto& th : pool) th.join();
  for (int r : rc) if (r) return r;
  return 0;
}

// Per-row thresholds (t, lo, hi) and the sizes of the sets U (at hi) and M
// (strictly between) as the reference's thresholds_<name> reports them through
// the iterators it returns.
template <typename Data, typename Result, typename Thr>
void store_thr(const Thr& t, const Data* base, const Data* end_unused,
               double* out_t, double* out_lo, double* out_hi, int64_t* nU,
               int64_t* nM) {
  (void)end_unused;
  *out_t = static_cast<double>(t.t);
  *out_lo = static_cast<double>(t.lo);
  *out_hi = static_cast<double>(t.hi);
  *nU = static_cast<int64_t>(t.first - base);
  *nM = static_cast<int64_t>(t.last - t.first);
}

template <typename Data, typename Result>
int run_thresholds(const std::string& name, const Data* a, idx_t m, idx_t n,
                   const ref_opts& o, double* t, double* lo_out, double* hi_out,
                   int64_t* nU, int64_t* nM) {
  using namespace sdca;
  std::vector<Data> aux_vec(static_cast<std::size_t>(m));
  Data* x = aux_vec.data();
  Data* xe = x + m;
  Result lo = static_cast<Result>(o.lo), hi = static_cast<Result>(o.hi);
  Result rhs = static_cast<Result>(o.rhs), rho = static_cast<Result>(o.rho);
  Result alpha = static_cast<Result>(o.alpha);
  idx_t k = static_cast<idx_t>(o.k), p = static_cast<idx_t>(o.p);
  const bool two = (name == "two_simplex" || name == "two_simplex_sort");
  for (idx_t r = 0; r < n; ++r) {
    std::copy(a + m * r, a + m * (r + 1), x);
    idx_t j = two ? 2 * r : r;
#define STORE(expr)                                                            \
  do {                                                                         \
    auto th = (expr);                                                          \
    store_thr<Data, Result>(th, x, xe, t + j, lo_out + j, hi_out + j, nU + j,  \
                            nM + j);                                           \
  } while (0)
    if (name == "knapsack" || name == "knapsack_eq") {
      STORE((thresholds_knapsack_eq<Result, Data*>(x, xe, lo, hi, rhs)));
    } else if (name == "knapsack_le") {
      STORE((thresholds_knapsack_le<Result, Data*>(x, xe, lo, hi, rhs)));
    } else if (name == "knapsack_le_biased") {
      STORE((thresholds_knapsack_le_biased<Result, Data*>(x, xe, lo, hi, rhs, rho)));
    } else if (name == "topk_simplex") {
      STORE((thresholds_topk_simplex<Result, Data*>(x, xe, k, rhs)));
    } else if (name == "topk_simplex_biased") {
      STORE((thresholds_topk_simplex_biased<Result, Data*>(x, xe, k, rhs, rho)));
    } else if (name == "topk_cone") {
      STORE((thresholds_topk_cone<Result, Data*>(x, xe, k)));
    } else if (name == "topk_cone_biased") {
      STORE((thresholds_topk_cone_biased<Result, Data*>(x, xe, k, rho)));
    } else if (name == "entropy") {
      STORE((thresholds_entropy<Result, Data*>(x, xe, hi, rhs)));
    } else if (name == "entropy_norm") {
      STORE((thresholds_entropy_norm<Result, Data*>(x, xe, hi, rhs)));
    } else if (name == "topk_entropy") {
      STORE((thresholds_topk_entropy<Result, Data*>(x, xe, k)));
    } else if (name == "topk_entropy_biased") {
      STORE((thresholds_topk_entropy_biased<Result, Data*>(x, xe, k, alpha)));
    } else if (two) {
      auto pr = (name == "two_simplex")
          ? thresholds_two_simplex<Result, Data*>(x, x + p, x + p, xe, rhs)
          : thresholds_two_simplex_sort<Result, Data*>(x, x + p, x + p, xe, rhs);
      store_thr<Data, Result>(pr.first, x, xe, t + j, lo_out + j, hi_out + j,
                              nU + j, nM + j);
      store_thr<Data, Result>(pr.second, x + p, xe, t + j + 1, lo_out + j + 1,
                              hi_out + j + 1, nU + j + 1, nM + j + 1);
    } else {
      return -1;
    }
#undef STORE
  }
  return 0;
}

// ---------------------------------------------------------------- eval -----
enum objective_id {
  OBJ_L2_ENTROPY = 0,            // softmax
  OBJ_L2_ENTROPY_TOPK,           // topk softmax
  OBJ_L2_HINGE_TOPK,             // top-k hinge alpha (gamma == 0)
  OBJ_L2_HINGE_TOPK_SMOOTH,      // top-k hinge alpha, smoothed
  OBJ_L2_TOPK_HINGE,             // top-k hinge beta / Crammer-Singer when k == 1
  OBJ_L2_TOPK_HINGE_SMOOTH,
  OBJ_L2_MULTILABEL_HINGE,
  OBJ_L2_MULTILABEL_HINGE_SMOOTH,
  OBJ_L2_MULTILABEL_ENTROPY
};

struct eval_args {
  int objective;
  double c, gamma;
  int64_t k;
  int input_kind;        // 0 = features (d x n), 1 = kernel (n_train x n)
  int64_t d;             // num_dimensions or num_train_examples
  int64_t n, m;
  const void* X;         // features or kernel matrix
  void* A;               // dual variables m x n (train: n == examples)
  void* W;               // primal variables d x m (features only)
  const void* W0;        // optional
  const int64_t* labels; // multiclass: n labels; multilabel: concatenated
  const int64_t* offsets;// multilabel: n + 1 offsets, else null
  int is_train;
  int nthreads;
  // fit only
  double epsilon;
  int64_t max_epoch, eval_epoch;
  int eval_on_start;
};

// out[0..6] = primal, dual, primal_loss, dual_loss, primal_regularizer,
//             dual_regularizer, rank_loss; accuracy has m entries (multiclass).
template <typename Result, typename Eval>
void store_eval_scalars(const Eval& e, double* out) {
  out[0] = static_cast<double>(e.primal);
  out[1] = static_cast<double>(e.dual);
  out[2] = static_cast<double>(e.primal_loss);
  out[3] = static_cast<double>(e.dual_loss);
  out[4] = static_cast<double>(e.primal_regularizer);
  out[5] = static_cast<double>(e.dual_regularizer);
}

template <typename Result>
void store_extra(const sdca::eval_train<Result, sdca::multiclass_output>& e,
                 double* out, double* acc) {
  out[6] = 0;
  for (std::size_t i = 0; i < e.accuracy.size(); ++i)
    acc[i] = static_cast<double>(e.accuracy[i]);
}
template <typename Result>
void store_extra(const sdca::eval_train<Result, sdca::multilabel_output>& e,
                 double* out, double*) {
  out[6] = static_cast<double>(e.rank_loss);
}
template <typename Result>
void store_test(const sdca::eval_test<Result, sdca::multiclass_output>& e,
                double* out, double* acc) {
  for (int i = 0; i < 7; ++i) out[i] = 0;
  out[2] = static_cast<double>(e.primal_loss);
  for (std::size_t i = 0; i < e.accuracy.size(); ++i)
    acc[i] = static_cast<double>(e.accuracy[i]);
}
template <typename Result>
void store_test(const sdca::eval_test<Result, sdca::multilabel_output>& e,
                double* out, double*) {
  for (int i = 0; i < 7; ++i) out[i] = 0;
  out[2] = static_cast<double>(e.primal_loss);
  out[6] = static_cast<double>(e.rank_loss);
}

inline sdca::multiclass_output make_out(const eval_args& a, sdca::multiclass_output*) {
  std::vector<sdca::size_type> v(a.labels, a.labels + a.n);
  return sdca::multiclass_output(static_cast<sdca::size_type>(a.m), v);
}
inline sdca::multilabel_output make_out(const eval_args& a, sdca::multilabel_output*) {
  std::vector<sdca::size_type> u(a.offsets, a.offsets + a.n + 1);
  std::vector<sdca::size_type> v(a.labels, a.labels + a.offsets[a.n]);
  sdca::validate_labels_and_offsets(static_cast<sdca::size_type>(a.m), v, u);
  return sdca::multilabel_output(static_cast<sdca::size_type>(a.m), v, u);
}

template <typename Data>
sdca::feature_input<Data> make_in(const eval_args& a, sdca::feature_input<Data>*) {
  return sdca::make_input_feature(static_cast<sdca::size_type>(a.d),
      static_cast<sdca::size_type>(a.n), static_cast<const Data*>(a.X));
}
template <typename Data>
sdca::kernel_input<Data> make_in(const eval_args& a, sdca::kernel_input<Data>*) {
  return sdca::make_input_kernel(static_cast<sdca::size_type>(a.d),
      static_cast<sdca::size_type>(a.n), static_cast<const Data*>(a.X));
}

template <typename Data, typename Result, template <typename> class Input,
          typename Output, template <typename, typename> class Objective>
sdca::solver_context<Data, Result, Input, Output, Objective>
build_context(const eval_args& a, Objective<Data, Result> obj,
              sdca::feature_input<Data>*) {
  auto ctx = sdca::make_context(make_in<Data>(a, (Input<Data>*)nullptr),
      make_out(a, (Output*)nullptr), std::move(obj),
      static_cast<Data*>(a.A), static_cast<Data*>(a.W));
  ctx.primal_initial = static_cast<const Data*>(a.W0);
  return ctx;
}
template <typename Data, typename Result, template <typename> class Input,
          typename Output, template <typename, typename> class Objective>
sdca::solver_context<Data, Result, Input, Output, Objective>
build_context(const eval_args& a, Objective<Data, Result> obj,
              sdca::kernel_input<Data>*) {
  return sdca::make_context(make_in<Data>(a, (Input<Data>*)nullptr),
      make_out(a, (Output*)nullptr), std::move(obj), static_cast<Data*>(a.A));
}

// The per-example body of evaluate_dataset (include/sdca/solver/eval.h:36-47),
// run over [i0, i1) into a private record, so that examples can be split over
// host threads for the timed baseline.  The reference itself is single
// threaded; with one thread evaluate_dataset is called directly instead.
template <typename Data, typename Result, typename Context, typename Eval>
void eval_range(Context& ctx, Eval& eval, sdca::size_type i0, sdca::size_type i1) {
  const sdca::size_type m = ctx.train.num_classes();
  std::vector<Data> sc(m);
  Data* scores = sc.data();
  for (sdca::size_type i = i0; i < i1; ++i) {
    Data* variables = ctx.dual_variables + m * i;
    sdca::eval_scores(i, m, ctx.train.in, ctx, scores);
    sdca::eval_regularizer_dual(m, ctx.train.in, ctx.objective, variables, scores, eval);
    sdca::eval_dual_loss(i, ctx.train.out, ctx.objective, variables, eval);
    sdca::eval_primal_loss(i, ctx.train.out, ctx.objective, scores, eval);
  }
}

template <typename Result>
void merge_init(sdca::eval_train<Result, sdca::multiclass_output>& e, sdca::size_type m) {
  e.accuracy.assign(m, Result());
}
template <typename Result>
void merge_init(sdca::eval_train<Result, sdca::multilabel_output>&, sdca::size_type) {}

template <typename Result>
void merge_extra(sdca::eval_train<Result, sdca::multiclass_output>& dst,
                 const sdca::eval_train<Result, sdca::multiclass_output>& src) {
  for (std::size_t i = 0; i < dst.accuracy.size(); ++i) dst.accuracy[i] += src.accuracy[i];
}
template <typename Result>
void merge_extra(sdca::eval_train<Result, sdca::multilabel_output>& dst,
                 const sdca::eval_train<Result, sdca::multilabel_output>& src) {
  dst.rank_loss += src.rank_loss;
}

template <typename Data, typename Result, template <typename> class Input,
          typename Output, template <typename, typename> class Objective>
int run_eval(const eval_args& a, Objective<Data, Result> obj, double* out, double* acc) {
  typedef sdca::solver_context<Data, Result, Input, Output, Objective> ctx_t;
  if (a.is_train) {
    ctx_t ctx = build_context<Data, Result, Input, Output, Objective>(
        a, std::move(obj), (Input<Data>*)nullptr);
    sdca::solver_scratch<Data, Input> scratch;
    scratch.scores.resize(static_cast<std::size_t>(a.m));
    if (a.nthreads <= 1) {
      sdca::evaluate_dataset(ctx, ctx.train, scratch);
    } else {
      const sdca::size_type m = ctx.train.num_classes(), n = ctx.train.num_examples();
      auto& eval = sdca::eval_begin(ctx.train);
      sdca::eval_recompute_primal(m, n, ctx.train, ctx);
      sdca::eval_regularizer_primal(m, ctx.train.in, ctx, eval);
      int T = a.nthreads;
      std::vector<typename ctx_t::train_eval_type> part(static_cast<std::size_t>(T));
      std::vector<std::thread> pool;
      for (int t = 0; t < T; ++t) {
        auto& pe = part[static_cast<std::size_t>(t)];
        merge_init(pe, m);
        sdca::size_type i0 = n * static_cast<sdca::size_type>(t) / static_cast<sdca::size_type>(T);
        sdca::size_type i1 = n * static_cast<sdca::size_type>(t + 1) / static_cast<sdca::size_type>(T);
        pool.emplace_back([&ctx, &pe, i0, i1]() {
          eval_range<Data, Result>(ctx, pe, i0, i1);
        });
      }
      for (auto& th : pool) th.join();
      for (auto& pe : part) {
        eval.primal_loss += pe.primal_loss;
        eval.dual_loss += pe.dual_loss;
        eval.primal_regularizer += pe.primal_regularizer;
        eval.dual_regularizer += pe.dual_regularizer;
        merge_extra(eval, pe);
      }
      sdca::eval_end(m, n, ctx, eval);
    }
    const auto& e = ctx.train.evals.back();
    store_eval_scalars<Result>(e, out);
    store_extra(e, out, acc);
  } else {
    // A held-out set: only primal loss and accuracy / rank loss are computed
    // (include/sdca/solver/eval/types.h:128-172).  The train set of the
    // context is a one-example stand-in that is never evaluated.
    eval_args tr = a;
    int64_t one_label = 0, one_off[2] = {0, 1};
    tr.n = 1; tr.labels = &one_label; tr.offsets = one_off;
    ctx_t ctx = build_context<Data, Result, Input, Output, Objective>(
        tr, std::move(obj), (Input<Data>*)nullptr);
    ctx.add_test(make_in<Data>(a, (Input<Data>*)nullptr), make_out(a, (Output*)nullptr));
    sdca::solver_scratch<Data, Input> scratch;
    scratch.scores.resize(static_cast<std::size_t>(a.m));
    sdca::evaluate_dataset(ctx, ctx.test[0], scratch);
    store_test(ctx.test[0].evals.back(), out, acc);
  }
  return 0;
}

// Held-out sets of the next fit (solver_context::add_test, context.h:87-91): set with
// sdca_ref_set_tests before sdca_ref_fit, cleared by the fit.  out receives, per
// evaluation e, {primal_loss, rank_loss} at out[2 * e ..]; acc the cumulative top-k
// accuracies (m per evaluation, multiclass).
struct ref_test_set {
  int64_t n;
  const void* X;
  const int64_t* labels;
  const int64_t* offsets;
  double* out;
  double* acc;
};
static std::vector<ref_test_set> g_tests;
static int64_t g_tests_cap = 0;

inline sdca::multiclass_output make_test_out(const ref_test_set& t, int64_t m, sdca::multiclass_output*) {
  std::vector<sdca::size_type> v(t.labels, t.labels + t.n);
  return sdca::multiclass_output(static_cast<sdca::size_type>(m), v);
}
inline sdca::multilabel_output make_test_out(const ref_test_set& t, int64_t m, sdca::multilabel_output*) {
  std::vector<sdca::size_type> u(t.offsets, t.offsets + t.n + 1);
  std::vector<sdca::size_type> v(t.labels, t.labels + t.offsets[t.n]);
  return sdca::multilabel_output(static_cast<sdca::size_type>(m), v, u);
}
template <typename Data>
sdca::feature_input<Data> make_test_in(const eval_args& a, const ref_test_set& t, sdca::feature_input<Data>*) {
  return sdca::make_input_feature(static_cast<sdca::size_type>(a.d), static_cast<sdca::size_type>(t.n),
                                  static_cast<const Data*>(t.X));
}
template <typename Data>
sdca::kernel_input<Data> make_test_in(const eval_args& a, const ref_test_set& t, sdca::kernel_input<Data>*) {
  return sdca::make_input_kernel(static_cast<sdca::size_type>(a.d), static_cast<sdca::size_type>(t.n),
                                 static_cast<const Data*>(t.X));
}
template <typename Result>
void store_test_eval(const sdca::eval_test<Result, sdca::multiclass_output>& e, double* out, double* acc, int64_t m) {
  out[0] = static_cast<double>(e.primal_loss); out[1] = 0;
  if (acc) for (int64_t j = 0; j < m && j < static_cast<int64_t>(e.accuracy.size()); ++j) acc[j] = static_cast<double>(e.accuracy[j]);
}
template <typename Result>
void store_test_eval(const sdca::eval_test<Result, sdca::multilabel_output>& e, double* out, double*, int64_t) {
  out[0] = static_cast<double>(e.primal_loss); out[1] = static_cast<double>(e.rank_loss);
}

// Fit: solver::solve with the given stopping criteria.  Returns the history of
// evaluations (7 doubles per evaluation) and the final status / epoch.
template <typename Data, typename Result, template <typename> class Input,
          typename Output, template <typename, typename> class Objective>
int run_fit(const eval_args& a, Objective<Data, Result> obj, double* hist,
            int64_t hist_cap, int64_t* num_evals, int64_t* epoch, int* status,
            double* acc_last) {
  auto ctx = build_context<Data, Result, Input, Output, Objective>(
      a, std::move(obj), (Input<Data>*)nullptr);
  ctx.criteria.epsilon = a.epsilon;
  ctx.criteria.max_epoch = static_cast<sdca::size_type>(a.max_epoch);
  ctx.criteria.eval_epoch = static_cast<sdca::size_type>(a.eval_epoch);
  ctx.criteria.eval_on_start = a.eval_on_start != 0;
  for (const ref_test_set& t : g_tests)
    ctx.add_test(make_test_in<Data>(a, t, (Input<Data>*)nullptr), make_test_out(t, a.m, (Output*)nullptr));
  auto solver = sdca::make_solver(ctx);
  solver.solve();
  for (std::size_t q = 0; q < g_tests.size(); ++q) {
    const auto& evs = ctx.test[q].evals;
    for (std::size_t e = 0; e < evs.size() && static_cast<int64_t>(e) < g_tests_cap; ++e)
      store_test_eval<Result>(evs[e], g_tests[q].out + 2 * e,
                              g_tests[q].acc ? g_tests[q].acc + a.m * static_cast<int64_t>(e) : nullptr, a.m);
  }
  g_tests.clear();
  int64_t ne = static_cast<int64_t>(ctx.train.evals.size());
  *num_evals = ne;
  for (int64_t i = 0; i < ne && i < hist_cap; ++i) {
    const auto& e = ctx.train.evals[static_cast<std::size_t>(i)];
    store_eval_scalars<Result>(e, hist + 8 * i);
    double extra[7] = {0, 0, 0, 0, 0, 0, 0};
    store_extra(e, extra, acc_last);
    hist[8 * i + 6] = extra[6];
    hist[8 * i + 7] = static_cast<double>(e.epoch);
  }
  *epoch = static_cast<int64_t>(ctx.epoch);
  *status = static_cast<int>(ctx.status);
  return 0;
}

template <typename Data, typename Result, template <typename> class Input, typename F>
int dispatch_objective(const eval_args& a, F&& f) {
  using namespace sdca;
  Result c = static_cast<Result>(a.c), g = static_cast<Result>(a.gamma);
  size_type k = static_cast<size_type>(a.k);
  switch (a.objective) {
    case OBJ_L2_ENTROPY:
      return f(make_objective_l2_entropy<Data, Result>(c), (multiclass_output*)nullptr);
    case OBJ_L2_ENTROPY_TOPK:
      return f(make_objective_l2_entropy_topk<Data, Result>(c, k), (multiclass_output*)nullptr);
    case OBJ_L2_HINGE_TOPK:
      return f(make_objective_l2_hinge_topk<Data, Result>(c, k), (multiclass_output*)nullptr);
    case OBJ_L2_HINGE_TOPK_SMOOTH:
      return f(make_objective_l2_hinge_topk_smooth<Data, Result>(c, g, k), (multiclass_output*)nullptr);
    case OBJ_L2_TOPK_HINGE:
      return f(make_objective_l2_topk_hinge<Data, Result>(c, k), (multiclass_output*)nullptr);
    case OBJ_L2_TOPK_HINGE_SMOOTH:
      return f(make_objective_l2_topk_hinge_smooth<Data, Result>(c, g, k), (multiclass_output*)nullptr);
    case OBJ_L2_MULTILABEL_HINGE:
      return f(make_objective_l2_multilabel_hinge<Data, Result>(c), (multilabel_output*)nullptr);
    case OBJ_L2_MULTILABEL_HINGE_SMOOTH:
      return f(make_objective_l2_multilabel_hinge_smooth<Data, Result>(c, g), (multilabel_output*)nullptr);
    case OBJ_L2_MULTILABEL_ENTROPY:
      return f(make_objective_l2_multilabel_entropy<Data, Result>(c), (multilabel_output*)nullptr);
  }
  return -3;
}

template <typename T> struct objective_traits;
template <typename D, typename R, template <typename, typename> class O>
struct objective_traits<O<D, R>> {
  template <template <typename> class Input, typename Output>
  static int eval(const eval_args& a, O<D, R> obj, double* out, double* acc) {
    return run_eval<D, R, Input, Output, O>(a, std::move(obj), out, acc);
  }
  template <template <typename> class Input, typename Output>
  static int fit(const eval_args& a, O<D, R> obj, double* hist, int64_t cap,
                 int64_t* ne, int64_t* ep, int* st, double* acc) {
    return run_fit<D, R, Input, Output, O>(a, std::move(obj), hist, cap, ne, ep, st, acc);
  }
};

template <typename Data, typename Result, template <typename> class Input>
int eval_dispatch(const eval_args& a, double* out, double* acc) {
  return dispatch_objective<Data, Result, Input>(a, [&](auto obj, auto* out_tag) {
    typedef typename std::remove_pointer<decltype(out_tag)>::type Output;
    typedef decltype(obj) Obj;
    return objective_traits<Obj>::template eval<Input, Output>(a, std::move(obj), out, acc);
  });
}

template <typename Data, typename Result, template <typename> class Input>
int fit_dispatch(const eval_args& a, double* hist, int64_t cap, int64_t* ne,
                 int64_t* ep, int* st, double* acc) {
  return dispatch_objective<Data, Result, Input>(a, [&](auto obj, auto* out_tag) {
    typedef typename std::remove_pointer<decltype(out_tag)>::type Output;
    typedef decltype(obj) Obj;
    return objective_traits<Obj>::template fit<Input, Output>(a, std::move(obj), hist, cap, ne, ep, st, acc);
  });
}

}  // namespace

extern "C" {

// dtype / result: 0 = float, 1 = double.
int sdca_ref_prox(const char* prox, int dtype, int result, void* a, int64_t m,
                  int64_t n, const ref_opts* o, int nthreads) {
  std::string name(prox);
  idx_t M = static_cast<idx_t>(m), N = static_cast<idx_t>(n);
  if (dtype == 0 && result == 0) return run_prox_threads<float, float>(name, (float*)a, M, N, *o, nthreads);
  if (dtype == 0 && result == 1) return run_prox_threads<float, double>(name, (float*)a, M, N, *o, nthreads);
  if (dtype == 1 && result == 0) return run_prox_threads<double, float>(name, (double*)a, M, N, *o, nthreads);
  if (dtype == 1 && result == 1) return run_prox_threads<double, double>(name, (double*)a, M, N, *o, nthreads);
  return -2;
}

int sdca_ref_thresholds(const char* prox, int dtype, int result, const void* a,
                        int64_t m, int64_t n, const ref_opts* o, double* t,
                        double* lo, double* hi, int64_t* nU, int64_t* nM) {
  std::string name(prox);
  idx_t M = static_cast<idx_t>(m), N = static_cast<idx_t>(n);
  if (dtype == 0 && result == 0) return run_thresholds<float, float>(name, (const float*)a, M, N, *o, t, lo, hi, nU, nM);
  if (dtype == 0 && result == 1) return run_thresholds<float, double>(name, (const float*)a, M, N, *o, t, lo, hi, nU, nM);
  if (dtype == 1 && result == 0) return run_thresholds<double, float>(name, (const double*)a, M, N, *o, t, lo, hi, nU, nM);
  if (dtype == 1 && result == 1) return run_thresholds<double, double>(name, (const double*)a, M, N, *o, t, lo, hi, nU, nM);
  return -2;
}

int sdca_ref_eval(const eval_args* a, int dtype, int result, double* out, double* acc) {
  sdca::logging::set_level(sdca::logging::level::none);
  try {
    if (a->input_kind == 0) {
      if (dtype == 0 && result == 0) return eval_dispatch<float, float, sdca::feature_input>(*a, out, acc);
      if (dtype == 0 && result == 1) return eval_dispatch<float, double, sdca::feature_input>(*a, out, acc);
      if (dtype == 1 && result == 0) return eval_dispatch<double, float, sdca::feature_input>(*a, out, acc);
      if (dtype == 1 && result == 1) return eval_dispatch<double, double, sdca::feature_input>(*a, out, acc);
    } else {
      if (dtype == 0 && result == 0) return eval_dispatch<float, float, sdca::kernel_input>(*a, out, acc);
      if (dtype == 0 && result == 1) return eval_dispatch<float, double, sdca::kernel_input>(*a, out, acc);
      if (dtype == 1 && result == 0) return eval_dispatch<double, float, sdca::kernel_input>(*a, out, acc);
      if (dtype == 1 && result == 1) return eval_dispatch<double, double, sdca::kernel_input>(*a, out, acc);
    }
  } catch (const std::exception&) {
    return -4;
  }
  return -2;
}

void sdca_ref_set_tests(const ref_test_set* sets, int count, int64_t cap) {
  g_tests.assign(sets, sets + count);
  g_tests_cap = cap;
}

int sdca_ref_fit(const eval_args* a, int dtype, int result, double* hist,
                 int64_t hist_cap, int64_t* num_evals, int64_t* epoch,
                 int* status, double* acc_last) {
  sdca::logging::set_level(sdca::logging::level::none);
  try {
    if (a->input_kind == 0) {
      if (dtype == 0 && result == 1) return fit_dispatch<float, double, sdca::feature_input>(*a, hist, hist_cap, num_evals, epoch, status, acc_last);
      if (dtype == 1 && result == 1) return fit_dispatch<double, double, sdca::feature_input>(*a, hist, hist_cap, num_evals, epoch, status, acc_last);
    } else {
      if (dtype == 0 && result == 1) return fit_dispatch<float, double, sdca::kernel_input>(*a, hist, hist_cap, num_evals, epoch, status, acc_last);
      if (dtype == 1 && result == 1) return fit_dispatch<double, double, sdca::kernel_input>(*a, hist, hist_cap, num_evals, epoch, status, acc_last);
    }
  } catch (const std::exception&) {
    return -4;
  }
  return -2;
}

// The example order of every epoch of solver::solve for n examples
// (include/sdca/solver.h:77-79,96-100): a default-seeded std::minstd_rand and
// std::shuffle applied cumulatively.  perm receives num_epochs * n indices.
int sdca_ref_epoch_permutations(int64_t n, int64_t num_epochs, int64_t* perm) {
  std::minstd_rand gen;
  gen.seed();
  std::vector<sdca::size_type> ex(static_cast<std::size_t>(n));
  for (int64_t i = 0; i < n; ++i) ex[static_cast<std::size_t>(i)] = static_cast<sdca::size_type>(i);
  for (int64_t e = 0; e < num_epochs; ++e) {
    std::shuffle(ex.begin(), ex.end(), gen);
    for (int64_t i = 0; i < n; ++i) perm[e * n + i] = static_cast<int64_t>(ex[static_cast<std::size_t>(i)]);
  }
  return 0;
}

// Scalar math of include/sdca/math/lambert.h:77-157 for known-answer checks.
double sdca_ref_lambert_w_exp_f64(double x) { return sdca::lambert_w_exp(x); }
float sdca_ref_lambert_w_exp_f32(float x) { return sdca::lambert_w_exp(x); }

}  // extern "C"
