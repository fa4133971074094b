// Test-only: the threshold routines of libsdca_b200/csrc compiled for the host
// with a lane group of one, so that the CPU test-suite can check their logic
// against the reference without a GPU.  Reductions are the identity here, so
// this exercises the algorithms, not the warp plumbing.  Never linked into the
// product library.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "../../include/sdca_b200.h"
#include "../../libsdca_b200/csrc/prox_core.cuh"
#include "../../libsdca_b200/csrc/prox_names.h"
#include "../../libsdca_b200/csrc/two_simplex_sort.cuh"

namespace {

template <typename Data, typename R>
int run(int prox, Data* a, int64_t m, int64_t n, const sdcab::ProxParams& q,
        sdcab_thresholds* thr, int apply) {
  using namespace sdcab;
  for (int64_t r = 0; r < n; ++r) {
    Data* x = a + r * m;
    if (prox == kLambertWExp) {
      if (apply) for (int64_t i = 0; i < m; ++i) x[i] = lambert_w_exp(x[i]);
      continue;
    }
    if (prox == kTwoSimplex) {
      StridedRow<Data> ra(x, q.p), rb(x + q.p, static_cast<int>(m) - q.p);
      ThrPair<R> pr = thr_two_simplex<R>(ra, rb, static_cast<R>(q.rhs));
      if (thr) {
        thr[2 * r] = {double(pr.a.t), double(pr.a.lo), double(pr.a.hi), pr.a.nU, pr.a.nM, thr_status(pr.a), 0};
        thr[2 * r + 1] = {double(pr.b.t), double(pr.b.lo), double(pr.b.hi), pr.b.nU, pr.b.nM, thr_status(pr.b), 0};
      }
      if (apply) {
        Applier<Data> fa(pr.a, kMapIdentity, 1.0), fb(pr.b, kMapIdentity, 1.0);
        for (int i = 0; i < q.p; ++i) x[i] = fa(x[i]);
        for (int64_t i = q.p; i < m; ++i) x[i] = fb(x[i]);
      }
      continue;
    }
    if (prox == kTwoSimplexSort) {
      const int na = q.p, nb = static_cast<int>(m) - q.p;
      std::vector<Data> sa(x, x + na), sb(x + na, x + m);
      std::sort(sa.begin(), sa.end(), std::greater<Data>());
      std::sort(sb.begin(), sb.end(), std::greater<Data>());
      R ta, tb; int rr, ss;
      two_simplex_sort_walk<R, Data>(sa.data(), na, sb.data(), nb, static_cast<R>(q.rhs), ta, tb, rr, ss);
      if (thr) {
        thr[2 * r] = {double(ta), 0.0, q.rhs, 0, rr, finite_(ta) ? 0 : 2, 0};
        thr[2 * r + 1] = {double(tb), 0.0, q.rhs, 0, ss, finite_(tb) ? 0 : 2, 0};
      }
      if (apply) {
        Applier<Data> fa(make_thr(ta, R(0), static_cast<R>(q.rhs), 0, 0, R(0), R(0)), kMapIdentity, 1.0);
        Applier<Data> fb(make_thr(tb, R(0), static_cast<R>(q.rhs), 0, 0, R(0), R(0)), kMapIdentity, 1.0);
        for (int i = 0; i < na; ++i) x[i] = fa(x[i]);
        for (int64_t i = na; i < m; ++i) x[i] = fb(x[i]);
      }
      continue;
    }
    StridedRow<Data> row(x, static_cast<int>(m));
    Thr<R> t = compute_thresholds<R>(prox, row, q);
    if (thr) thr[r] = {double(t.t), double(t.lo), double(t.hi), t.nU, t.nM, thr_status(t), 0};
    if (apply) {
      Applier<Data> f(t, prox_map(prox), q.alpha);
      for (int64_t i = 0; i < m; ++i) x[i] = f(x[i]);
    }
  }
  return 0;
}

}  // namespace

extern "C" int sdcab_hostsim_prox(const char* name, int dtype, void* a, int64_t m,
                                  int64_t n, const sdcab_prox_opts* o,
                                  sdcab_thresholds* thr, int apply) {
  int prox = sdcab::prox_id_from_name(name);
  if (prox < 0) return SDCAB_ERR_PROX;
  sdcab::ProxParams q{o->lo, o->hi, o->rhs, o->rho, o->alpha, (int)o->k, (int)o->p, o->accurate_math ? 1 : 0};
  const bool f = (o->precision == SDCAB_PRECISION_FLOAT);
  if (dtype == 0) return f ? run<float, float>(prox, (float*)a, m, n, q, thr, apply)
                           : run<float, double>(prox, (float*)a, m, n, q, thr, apply);
  return f ? run<double, float>(prox, (double*)a, m, n, q, thr, apply)
           : run<double, double>(prox, (double*)a, m, n, q, thr, apply);
}

// ---- evaluation: the per-example loss code of losses.cuh with one lane -------
#include <vector>

#include "../../libsdca_b200/csrc/eval_host.h"

namespace {

template <typename Data, typename R>
int run_eval(const sdcab_objective* obj, const sdcab_problem* p, double* sums) {
  using namespace sdcab;
  const ObjectiveParams q = to_params(obj);
  const int m = static_cast<int>(p->m);
  const long long n = p->n, d = p->d;
  const Data* X = static_cast<const Data*>(p->x);
  const Data* A = static_cast<const Data*>(p->a);
  const Data* W = static_cast<const Data*>(p->w);
  const Data* W0 = static_cast<const Data*>(p->w0);
  for (int i = 0; i < SDCAB_EVAL_SUMS(m); ++i) sums[i] = 0;
  sums[5] = static_cast<double>(n);
  if (p->is_train && p->input_kind == SDCAB_INPUT_FEATURES && p->include_primal_regularizer) {
    double ww = 0, w0w = 0;
    for (long long i = 0; i < d * m; ++i) {
      ww += double(W[i]) * double(W[i]);
      if (W0) w0w += double(W0[i]) * double(W[i]);
    }
    sums[2] += W0 ? ww / 2 - w0w : ww / 2;
    sums[3] += ww / 2;
  }
  std::vector<Data> s(m);
  std::vector<unsigned> mask((m + 31) / 32);
  const bool ml = objective_is_multilabel(q.id);
  for (long long e = 0; e < n; ++e) {
    for (int j = 0; j < m; ++j) {
      Data acc = 0;
      if (p->input_kind == SDCAB_INPUT_FEATURES) {
        for (long long l = 0; l < d; ++l) acc = std::fma(X[e * d + l], W[j * d + l], acc);
      } else {
        for (long long l = 0; l < d; ++l) acc = std::fma(X[e * d + l], A[l * m + j], acc);
      }
      s[j] = acc;
    }
    const Data* a = (p->is_train && A) ? A + (p->a_row_offset + e) * m : nullptr;
    if (!ml) {
      const int y = static_cast<int>(p->labels[e]);
      int rank;
      sums[0] += double(multiclass_primal_loss<R, Data>(q, s.data(), m, y, rank));
      sums[8 + rank] += 1;
      if (a) sums[1] += double(multiclass_dual_loss<R, Data>(q, a, m, y));
    } else {
      const long long off = p->offsets[e];
      const int nl = static_cast<int>(p->offsets[e + 1] - off);
      std::fill(mask.begin(), mask.end(), 0u);
      for (int g = 0; g < nl; ++g) mask[p->labels[off + g] >> 5] |= 1u << (p->labels[off + g] & 31);
      R rl;
      sums[0] += double(multilabel_primal_loss<R, Data>(
          q, s.data(), m, mask.data(), reinterpret_cast<const long long*>(p->labels + off), nl, rl));
      sums[4] += double(rl);
      if (a) sums[1] += double(multilabel_dual_loss<R, Data>(q, a, m, mask.data(), nl));
    }
    if (a && p->input_kind == SDCAB_INPUT_KERNEL) {
      R dot = 0;
      for (int j = 0; j < m; ++j) dot += R(a[j]) * R(s[j]);
      sums[2] += double(dot) * 0.5; sums[3] += double(dot) * 0.5;
    }
  }
  return 0;
}

}  // namespace

extern "C" int sdcab_hostsim_eval(const sdcab_objective* obj, const sdcab_problem* p, int dtype,
                                  double* sums) {
  const bool f = (obj->precision == SDCAB_PRECISION_FLOAT);
  if (dtype == 0) return f ? run_eval<float, float>(obj, p, sums) : run_eval<float, double>(obj, p, sums);
  return f ? run_eval<double, float>(obj, p, sums) : run_eval<double, double>(obj, p, sums);
}

extern "C" int sdcab_hostsim_eval_finish(const sdcab_objective* obj, int64_t m, const double* sums,
                                         sdcab_eval_record* rec, double* acc) {
  return sdcab::eval_finish(obj, m, sums, rec, acc);
}

extern "C" int sdcab_hostsim_objective_from_name(const char* name, double c, double gamma,
                                                 int64_t k, sdcab_objective* out) {
  return sdcab::objective_from_name(name, c, gamma, k, out);
}

// ---- fit: the device code's update step with one lane, driven by the host-side
// epoch order and stopping rule the library uses ---------------------------------
#include <chrono>
#include <ctime>
#include "../../libsdca_b200/csrc/fit_host.h"
#include "../../libsdca_b200/csrc/per_device.h"
#include "../../libsdca_b200/csrc/update_core.cuh"

namespace {

template <typename Data, typename R>
int run_fit(const sdcab_objective* obj, const sdcab_problem* p, const sdcab_fit_criteria* crit,
            const int64_t* permutations, sdcab_eval_record* evals, int64_t cap,
            sdcab_fit_result* res) {
  using namespace sdcab;
  const ObjectiveParams q = to_params(obj);
  const int m = static_cast<int>(p->m);
  const long long n = p->n, d = p->d;
  const Data* X = static_cast<const Data*>(p->x);
  Data* A = static_cast<Data*>(const_cast<void*>(p->a));
  Data* W = static_cast<Data*>(const_cast<void*>(p->w));
  const bool kernel = (p->input_kind == SDCAB_INPUT_KERNEL);
  std::vector<Data> s(m), v(m), old(m);
  std::vector<double> sums(SDCAB_EVAL_SUMS(m));
  std::vector<sdcab_eval_record> hist;
  sdcab_problem ep = *p;
  ep.is_train = 1; ep.a_row_offset = 0; ep.include_primal_regularizer = 1;
  auto evaluate = [&]() {
    run_eval<Data, R>(obj, &ep, sums.data());
    sdcab_eval_record rec;
    eval_finish(obj, m, sums.data(), &rec, nullptr);
    hist.push_back(rec);
    if (evals && (int64_t)hist.size() <= cap) evals[hist.size() - 1] = rec;
  };
  const double eps_floor = std::max(double(num<Data>::eps()), double(num<R>::eps()));
  const std::clock_t cpu_begin = std::clock();
  const auto wall_begin = std::chrono::steady_clock::now();
  auto check = [&](int st, int64_t epoch) {
    const double cpu = double(std::clock() - cpu_begin) / CLOCKS_PER_SEC;
    const double wall = std::chrono::duration<double>(std::chrono::steady_clock::now() - wall_begin).count();
    return check_stopping(st, hist.empty() ? nullptr : &hist.back(),
                          hist.size() > 1 ? &hist[hist.size() - 2] : nullptr, crit->epsilon,
                          epoch, crit->max_epoch, eps_floor, crit->max_cpu_time, cpu,
                          crit->max_wall_time, wall);
  };
  int64_t epoch = 0;
  int status = crit->max_epoch > 0 ? SDCAB_FIT_SOLVING : SDCAB_FIT_MAX_EPOCH;
  bool evaluated = false;
  if (crit->eval_on_start) { evaluate(); status = check(status, epoch); }
  MinstdRand gen;
  std::vector<int64_t> order(n);
  for (long long i = 0; i < n; ++i) order[i] = i;
  while (status == SDCAB_FIT_SOLVING) {
    evaluated = false;
    const int64_t* ord;
    if (permutations) ord = permutations + epoch * n;
    else { shuffle_like_libstdcxx(order, gen); ord = order.data(); }
    for (long long step = 0; step < n; ++step) {
      const long long i = ord[step];
      Data norm2;
      if (kernel) {
        norm2 = X[n * i + i];
      } else {
        double t = 0;
        for (long long r = 0; r < d; ++r) t = std::fma(double(X[d * i + r]), double(X[d * i + r]), t);
        norm2 = Data(t);
      }
      if (!(norm2 > 0)) continue;
      for (int j = 0; j < m; ++j) {
        double acc = 0;
        if (kernel) for (long long l = 0; l < n; ++l) acc = std::fma(double(A[l * m + j]), double(X[n * i + l]), acc);
        else for (long long r = 0; r < d; ++r) acc = std::fma(double(W[d * j + r]), double(X[d * i + r]), acc);
        s[j] = Data(acc);
      }
      Data* a = A + i * m;
      for (int j = 0; j < m; ++j) old[j] = a[j];
      if (objective_is_multilabel(q.id)) {
        const long long off = p->offsets[i];
        const int nl = static_cast<int>(p->offsets[i + 1] - off);
        std::vector<unsigned> mask((m + 31) / 32, 0u);
        for (int g = 0; g < nl; ++g) mask[p->labels[off + g] >> 5] |= 1u << (p->labels[off + g] & 31);
        update_dual_variables_multilabel_hinge<R, Data>(q, norm2, s.data(), a, v.data(), m, mask.data(), nl);
      } else {
        update_dual_variables_multiclass<R, Data>(q, norm2, s.data(), a, v.data(), m, (int)p->labels[i]);
      }
      if (!kernel) {
        Data asum = 0;
        for (int j = 0; j < m; ++j) { old[j] -= a[j]; asum += abs_(old[j]); }
        if (asum > num<Data>::eps())
          for (int j = 0; j < m; ++j)
            for (long long r = 0; r < d; ++r) W[d * j + r] = W[d * j + r] - X[d * i + r] * old[j];
      }
    }
    ++epoch;
    if (crit->eval_epoch > 0 && epoch % crit->eval_epoch == 0) { evaluate(); evaluated = true; }
    status = check(status, epoch);
  }
  if (!evaluated && !(crit->eval_on_start && epoch == 0)) evaluate();
  res->status = status; res->epoch = epoch; res->num_evals = (int64_t)hist.size();
  res->solve_seconds = 0; res->eval_seconds = 0;
  res->cpu_seconds = double(std::clock() - cpu_begin) / CLOCKS_PER_SEC;
  res->wall_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - wall_begin).count();
  return 0;
}

}  // namespace

extern "C" int sdcab_hostsim_fit(const sdcab_objective* obj, const sdcab_problem* p, int dtype,
                                 const sdcab_fit_criteria* crit, const int64_t* permutations,
                                 sdcab_eval_record* evals, int64_t cap, sdcab_fit_result* res) {
  if (!sdcab::objective_has_update(obj->id)) return SDCAB_ERR_NOT_IMPLEMENTED;
  const bool f = (obj->precision == SDCAB_PRECISION_FLOAT);
  if (dtype == 0) return f ? run_fit<float, float>(obj, p, crit, permutations, evals, cap, res)
                           : run_fit<float, double>(obj, p, crit, permutations, evals, cap, res);
  return f ? run_fit<double, float>(obj, p, crit, permutations, evals, cap, res)
           : run_fit<double, double>(obj, p, crit, permutations, evals, cap, res);
}

extern "C" int sdcab_hostsim_epoch_permutations(int64_t n, int64_t epochs, int64_t* perm) {
  sdcab::epoch_permutations(n, epochs, perm);
  return 0;
}

// The library's stopping rule and label checks, as they are (host code).
extern "C" int sdcab_hostsim_check_stopping(int status, const sdcab_eval_record* last,
                                            const sdcab_eval_record* before, double epsilon,
                                            int64_t epoch, int64_t max_epoch, double data_epsilon,
                                            double max_cpu, double cpu_now, double max_wall,
                                            double wall_now) {
  return sdcab::check_stopping(status, last, before, epsilon, epoch, max_epoch, data_epsilon, max_cpu,
                               cpu_now, max_wall, wall_now);
}

extern "C" int sdcab_hostsim_validate_labels(const int64_t* labels, const int64_t* offsets, int64_t n,
                                             int64_t m, int multilabel) {
  return sdcab::validate_labels(labels, offsets, n, m, multilabel != 0);
}

// Per-device bookkeeping: visits the devices in `order` and reports, for each
// visit, whether it was the first one on that device (bit i of the result).
extern "C" uint64_t sdcab_hostsim_once_per_device(const int* order, int count) {
  sdcab::OncePerDevice once;
  uint64_t bits = 0;
  for (int i = 0; i < count && i < 64; ++i)
    if (once.first_time(order[i])) bits |= uint64_t(1) << i;
  return bits;
}
