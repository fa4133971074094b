// Test-only: the threshold routines of libsdca_b200/csrc compiled for the host
// with a lane group of one, so that the CPU test-suite can check their logic
// against the reference without a GPU.  Reductions are the identity here, so
// this exercises the algorithms, not the warp plumbing.  Never linked into the
// product library.
#include <cstdint>
#include <cstring>
#include <string>

#include "../../include/sdca_b200.h"
#include "../../libsdca_b200/csrc/prox_core.cuh"
#include "../../libsdca_b200/csrc/prox_names.h"

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
        thr[2 * r] = {double(pr.a.t), double(pr.a.lo), double(pr.a.hi), pr.a.nU, pr.a.nM};
        thr[2 * r + 1] = {double(pr.b.t), double(pr.b.lo), double(pr.b.hi), pr.b.nU, pr.b.nM};
      }
      if (apply) {
        Applier<Data> fa(pr.a, kMapIdentity, 1.0), fb(pr.b, kMapIdentity, 1.0);
        for (int i = 0; i < q.p; ++i) x[i] = fa(x[i]);
        for (int64_t i = q.p; i < m; ++i) x[i] = fb(x[i]);
      }
      continue;
    }
    StridedRow<Data> row(x, static_cast<int>(m));
    Thr<R> t = compute_thresholds<R>(prox, row, q);
    if (thr) thr[r] = {double(t.t), double(t.lo), double(t.hi), t.nU, t.nM};
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
  sdcab::ProxParams q{o->lo, o->hi, o->rhs, o->rho, o->alpha, (int)o->k, (int)o->p};
  const bool f = (o->precision == SDCAB_PRECISION_FLOAT);
  if (dtype == 0) return f ? run<float, float>(prox, (float*)a, m, n, q, thr, apply)
                           : run<float, double>(prox, (float*)a, m, n, q, thr, apply);
  return f ? run<double, float>(prox, (double*)a, m, n, q, thr, apply)
           : run<double, double>(prox, (double*)a, m, n, q, thr, apply);
}
