/*
 * Test infrastructure: a small sequential CBLAS used only by the CPU oracle.
 *
 * The reference solver calls an external CBLAS (include/sdca/math/blas.h:33-415
 * of the reference).  No BLAS version is pinned by the reference, so the oracle
 * links these plain loops to get results that do not depend on a threaded
 * library.  Every routine accumulates in the precision of its arguments and in
 * index order, like the netlib reference BLAS.  Column-major, any stride.
 *
 * For the timed CPU baseline the vector/matrix kernels can be redirected at run
 * time to an optimised CBLAS found on the machine (sdca_ref_use_blas).
 */
#include <dlfcn.h>
#include <math.h>
#include <stddef.h>
#include <stdio.h>

enum { ColMajor = 102, NoTrans = 111 };

typedef void (*sgemv_fn)(int, int, int, int, float, const float*, int,
                         const float*, int, float, float*, int);
typedef void (*dgemv_fn)(int, int, int, int, double, const double*, int,
                         const double*, int, double, double*, int);
typedef void (*sgemm_fn)(int, int, int, int, int, int, float, const float*, int,
                         const float*, int, float, float*, int);
typedef void (*dgemm_fn)(int, int, int, int, int, int, double, const double*,
                         int, const double*, int, double, double*, int);

static sgemv_fn ext_sgemv;
static dgemv_fn ext_dgemv;
static sgemm_fn ext_sgemm;
static dgemm_fn ext_dgemm;

/* Redirect gemv/gemm to an external CBLAS; returns 0 on success. */
int sdca_ref_use_blas(const char* path, int num_threads) {
  if (!path) { ext_sgemv = 0; ext_dgemv = 0; ext_sgemm = 0; ext_dgemm = 0; return 0; }
  void* h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) { fprintf(stderr, "sdca_ref_use_blas: %s\n", dlerror()); return -1; }
  void (*set_threads)(int) = (void (*)(int))dlsym(h, "openblas_set_num_threads");
  if (set_threads && num_threads > 0) set_threads(num_threads);
  ext_sgemv = (sgemv_fn)dlsym(h, "cblas_sgemv");
  ext_dgemv = (dgemv_fn)dlsym(h, "cblas_dgemv");
  ext_sgemm = (sgemm_fn)dlsym(h, "cblas_sgemm");
  ext_dgemm = (dgemm_fn)dlsym(h, "cblas_dgemm");
  return (ext_sgemv && ext_dgemv && ext_sgemm && ext_dgemm) ? 0 : -2;
}

#define LEVEL1(P, T)                                                           \
  void cblas_##P##scal(int n, T a, T* x, int ix) {                             \
    for (int i = 0; i < n; ++i) x[(ptrdiff_t)i * ix] *= a;                     \
  }                                                                            \
  void cblas_##P##copy(int n, const T* x, int ix, T* y, int iy) {              \
    for (int i = 0; i < n; ++i) y[(ptrdiff_t)i * iy] = x[(ptrdiff_t)i * ix];   \
  }                                                                            \
  void cblas_##P##swap(int n, T* x, int ix, T* y, int iy) {                    \
    for (int i = 0; i < n; ++i) {                                              \
      T v = x[(ptrdiff_t)i * ix];                                              \
      x[(ptrdiff_t)i * ix] = y[(ptrdiff_t)i * iy];                             \
      y[(ptrdiff_t)i * iy] = v;                                                \
    }                                                                          \
  }                                                                            \
  void cblas_##P##axpy(int n, T a, const T* x, int ix, T* y, int iy) {         \
    for (int i = 0; i < n; ++i) y[(ptrdiff_t)i * iy] += a * x[(ptrdiff_t)i * ix]; \
  }                                                                            \
  T cblas_##P##dot(int n, const T* x, int ix, const T* y, int iy) {            \
    T s = 0;                                                                   \
    for (int i = 0; i < n; ++i) s += x[(ptrdiff_t)i * ix] * y[(ptrdiff_t)i * iy]; \
    return s;                                                                  \
  }                                                                            \
  T cblas_##P##asum(int n, const T* x, int ix) {                               \
    T s = 0;                                                                   \
    for (int i = 0; i < n; ++i) s += (T)fabs((double)x[(ptrdiff_t)i * ix]);    \
    return s;                                                                  \
  }                                                                            \
  T cblas_##P##nrm2(int n, const T* x, int ix) {                               \
    double s = 0;                                                              \
    for (int i = 0; i < n; ++i) {                                              \
      double v = (double)x[(ptrdiff_t)i * ix];                                 \
      s += v * v;                                                              \
    }                                                                          \
    return (T)sqrt(s);                                                         \
  }                                                                            \
  void cblas_##P##ger(int order, int m, int n, T alpha, const T* x, int ix,    \
                      const T* y, int iy, T* a, int lda) {                     \
    (void)order;                                                               \
    for (int j = 0; j < n; ++j) {                                              \
      T t = alpha * y[(ptrdiff_t)j * iy];                                      \
      T* col = a + (ptrdiff_t)j * lda;                                         \
      for (int i = 0; i < m; ++i) col[i] += x[(ptrdiff_t)i * ix] * t;          \
    }                                                                          \
  }

LEVEL1(s, float)
LEVEL1(d, double)

#define GEMV(P, T, EXT)                                                        \
  void cblas_##P##gemv(int order, int trans, int m, int n, T alpha,            \
                       const T* a, int lda, const T* x, int ix, T beta, T* y,  \
                       int iy) {                                               \
    if (EXT) { EXT(order, trans, m, n, alpha, a, lda, x, ix, beta, y, iy); return; } \
    int leny = (trans == NoTrans) ? m : n;                                     \
    for (int i = 0; i < leny; ++i) {                                           \
      T* yi = y + (ptrdiff_t)i * iy;                                           \
      *yi = (beta == (T)0) ? (T)0 : beta * *yi;                                \
    }                                                                          \
    if (trans == NoTrans) {                                                    \
      for (int j = 0; j < n; ++j) {                                            \
        T t = alpha * x[(ptrdiff_t)j * ix];                                    \
        const T* col = a + (ptrdiff_t)j * lda;                                 \
        for (int i = 0; i < m; ++i) y[(ptrdiff_t)i * iy] += t * col[i];        \
      }                                                                        \
    } else {                                                                   \
      for (int j = 0; j < n; ++j) {                                            \
        const T* col = a + (ptrdiff_t)j * lda;                                 \
        T s = 0;                                                               \
        for (int i = 0; i < m; ++i) s += col[i] * x[(ptrdiff_t)i * ix];        \
        y[(ptrdiff_t)j * iy] += alpha * s;                                     \
      }                                                                        \
    }                                                                          \
  }

GEMV(s, float, ext_sgemv)
GEMV(d, double, ext_dgemv)

#define GEMM(P, T, EXT)                                                        \
  void cblas_##P##gemm(int order, int ta, int tb, int m, int n, int k,         \
                       T alpha, const T* a, int lda, const T* b, int ldb,      \
                       T beta, T* c, int ldc) {                                \
    if (EXT) { EXT(order, ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc); return; } \
    for (int j = 0; j < n; ++j) {                                              \
      T* cj = c + (ptrdiff_t)j * ldc;                                          \
      for (int i = 0; i < m; ++i) cj[i] = (beta == (T)0) ? (T)0 : beta * cj[i]; \
      for (int l = 0; l < k; ++l) {                                            \
        T bv = (tb == NoTrans) ? b[(ptrdiff_t)j * ldb + l]                     \
                               : b[(ptrdiff_t)l * ldb + j];                    \
        T t = alpha * bv;                                                      \
        if (ta == NoTrans) {                                                   \
          const T* al = a + (ptrdiff_t)l * lda;                                \
          for (int i = 0; i < m; ++i) cj[i] += t * al[i];                      \
        } else {                                                               \
          for (int i = 0; i < m; ++i) cj[i] += t * a[(ptrdiff_t)i * lda + l];  \
        }                                                                      \
      }                                                                        \
    }                                                                          \
  }

GEMM(s, float, ext_sgemm)
GEMM(d, double, ext_dgemm)
