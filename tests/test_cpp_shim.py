"""The header-only C++ shim (include/sdca_b200.hpp): a small C++ program written the
way a caller of the reference's headers is written (same function names, same
argument order, host pointers) is compiled against the C ABI.  Without a GPU the
test stops at compiling and linking; on a GPU the program really runs and its
results are compared with the reference's."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SOURCE = r'''
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "sdca_b200.hpp"

template <typename T>
static std::vector<T> read_all(const char* path) {
  std::FILE* f = std::fopen(path, "rb");
  if (!f) { std::perror(path); std::exit(2); }
  std::fseek(f, 0, SEEK_END); long bytes = std::ftell(f); std::fseek(f, 0, SEEK_SET);
  std::vector<T> v(static_cast<size_t>(bytes) / sizeof(T));
  if (std::fread(v.data(), sizeof(T), v.size(), f) != v.size()) std::exit(3);
  std::fclose(f);
  return v;
}
template <typename T>
static void write_all(const char* path, const std::vector<T>& v) {
  std::FILE* f = std::fopen(path, "wb");
  std::fwrite(v.data(), sizeof(T), v.size(), f);
  std::fclose(f);
}

// argv: dir m_prox n d m   (files in dir: rows_f32.bin rows_f64.bin X.bin labels.bin A.bin W.bin)
int main(int argc, char** argv) {
  if (argc < 6) return 0;   // compile-and-link check only
  const std::string dir = argv[1];
  const std::ptrdiff_t mp = std::atol(argv[2]);
  const int64_t n = std::atol(argv[3]), d = std::atol(argv[4]), m = std::atol(argv[5]);
  try {
    // batched prox, the reference's call shape: (dim, first, last, aux, params...)
    std::vector<float> a = read_all<float>((dir + "/rows_f32.bin").c_str()), aux(mp);
    std::vector<float> a2 = a;
    sdca::b200::prox_topk_simplex(mp, a.data(), a.data() + a.size(), aux.data(), 3, 1.0);
    write_all((dir + "/out_topk_simplex.bin").c_str(), a);
    sdca::b200::prox_topk_cone<float>(mp, a2.data(), a2.data() + a2.size(), aux.data(), 3);
    write_all((dir + "/out_topk_cone.bin").c_str(), a2);
    std::vector<double> b = read_all<double>((dir + "/rows_f64.bin").c_str());
    std::vector<double> b2 = b, b3 = b, b4 = b;
    sdca::b200::prox_knapsack_eq(mp, b.data(), b.data() + b.size(), b.data());
    write_all((dir + "/out_knapsack_eq.bin").c_str(), b);
    sdca::b200::prox_two_simplex(mp, 3, b2.data(), b2.data() + b2.size(), b2.data(), 1.0);
    write_all((dir + "/out_two_simplex.bin").c_str(), b2);
    sdca::b200::prox_two_simplex_sort(mp, 3, b4.data(), b4.data() + b4.size(), b4.data(), 1.0);
    write_all((dir + "/out_two_simplex_sort.bin").c_str(), b4);
    sdca::b200::apply_lambert_w_exp(mp, b3.data(), b3.data() + b3.size());
    write_all((dir + "/out_lambert.bin").c_str(), b3);

    // evaluate_dataset and solve on a small feature problem
    std::vector<double> X = read_all<double>((dir + "/X.bin").c_str());
    std::vector<int64_t> labels = read_all<int64_t>((dir + "/labels.bin").c_str());
    std::vector<double> A = read_all<double>((dir + "/A.bin").c_str());
    std::vector<double> W = read_all<double>((dir + "/W.bin").c_str());
    sdcab_objective o;
    sdca::b200::check(sdcab_objective_from_name("msvm_smooth", 1.0, 1.0, 1, &o), "objective");
    sdcab_problem p = sdcab_problem();
    p.input_kind = SDCAB_INPUT_FEATURES; p.is_train = 1; p.d = d; p.n = n; p.m = m;
    p.x = X.data(); p.a = A.data(); p.w = W.data(); p.labels = labels.data();
    p.include_primal_regularizer = 1;
    std::vector<double> acc;
    sdcab_eval_record rec = sdca::b200::evaluate_dataset<double>(o, p, &acc);
    std::vector<double> out_eval = {rec.primal, rec.dual, rec.primal_loss, rec.dual_loss,
                                    rec.primal_regularizer, rec.dual_regularizer, acc[0]};
    write_all((dir + "/out_eval.bin").c_str(), out_eval);

    std::vector<double> A0(A.size(), 0.0), W0(W.size(), 0.0);
    p.a = A0.data(); p.w = W0.data();
    sdcab_fit_criteria c = sdcab_fit_criteria();
    c.epsilon = 1e-3; c.max_epoch = 100; c.eval_epoch = 10;
    std::vector<sdcab_eval_record> evals;
    sdcab_fit_result r = sdca::b200::solve<double>(o, p, c, &evals);
    std::vector<double> out_fit = {static_cast<double>(r.status), static_cast<double>(r.epoch),
                                   static_cast<double>(evals.size()), evals.back().primal,
                                   evals.back().dual};
    write_all((dir + "/out_fit.bin").c_str(), out_fit);
    write_all((dir + "/out_fit_A.bin").c_str(), A0);

    // errors surface as exceptions carrying the LIBSDCA:* identifier
    try {
      sdca::b200::prox_topk_simplex(mp, a.data(), a.data() + a.size(), aux.data(), mp + 1, 1.0);
      return 4;
    } catch (const std::runtime_error& e) {
      if (std::string(e.what()).find("LIBSDCA:arg_range") == std::string::npos) return 5;
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "%s\n", e.what());
    return 1;
  }
  return 0;
}
'''


def build_program(tmp):
    import libsdca_b200
    lib = libsdca_b200.library_path()
    if not os.path.exists(lib):
        pytest.skip("library not built")
    src = os.path.join(tmp, "shim.cpp")
    open(src, "w").write(SOURCE)
    exe = os.path.join(tmp, "shim")
    cmd = ["g++", "-std=c++11", "-I", os.path.join(ROOT, "include"), src, "-o", exe, lib,
           "-Wl,-rpath," + os.path.dirname(lib), "-Wl,-rpath,/usr/local/cuda/lib64"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_shim_compiles_and_links():
    with tempfile.TemporaryDirectory() as tmp:
        build_program(tmp)


@pytest.mark.gpu
def test_shim_program_matches_reference(ref, cuda_lib):
    rng = np.random.default_rng(31)
    mp, rows = 12, 64
    n, d, m = 240, 10, 6
    rows32 = rng.standard_normal((rows, mp)).astype(np.float32)
    rows64 = rng.standard_normal((rows, mp))
    means = rng.standard_normal((m, d)) * 2
    labels = rng.integers(0, m, n).astype(np.int64)
    X = means[labels] + rng.standard_normal((n, d))
    A = -np.abs(rng.standard_normal((n, m))) * 0.01
    A[np.arange(n), labels] = 0.02
    W = A.T @ X
    with tempfile.TemporaryDirectory() as tmp:
        exe = build_program(tmp)
        for name, arr in (("rows_f32", rows32), ("rows_f64", rows64), ("X", X), ("labels", labels),
                          ("A", A), ("W", W)):
            np.ascontiguousarray(arr).tofile(os.path.join(tmp, name + ".bin"))
        res = subprocess.run([exe, tmp, str(mp), str(n), str(d), str(m)], capture_output=True, text=True)
        assert res.returncode == 0, (res.returncode, res.stderr)
        load = lambda name, dt: np.fromfile(os.path.join(tmp, name + ".bin"), dtype=dt)
        got = {
            "topk_simplex": load("out_topk_simplex", np.float32).reshape(rows, mp),
            "topk_cone": load("out_topk_cone", np.float32).reshape(rows, mp),
            "knapsack_eq": load("out_knapsack_eq", np.float64).reshape(rows, mp),
            "two_simplex": load("out_two_simplex", np.float64).reshape(rows, mp),
            "two_simplex_sort": load("out_two_simplex_sort", np.float64).reshape(rows, mp),
            "lambert": load("out_lambert", np.float64).reshape(rows, mp),
        }
        out_eval = load("out_eval", np.float64)
        out_fit = load("out_fit", np.float64)
        fit_A = load("out_fit_A", np.float64).reshape(n, m)
    scale32 = np.maximum(1, np.abs(rows32).max(axis=1, keepdims=True))
    assert (np.abs(got["topk_simplex"] - ref.prox("topk_simplex", rows32, k=3, rhs=1.0)) <= 1e-5 * scale32).all()
    assert (np.abs(got["topk_cone"] - ref.prox("topk_cone", rows32, k=3)) <= 1e-5 * scale32).all()
    scale64 = np.maximum(1, np.abs(rows64).max(axis=1, keepdims=True))
    assert (np.abs(got["knapsack_eq"] - ref.prox("knapsack_eq", rows64)) <= 1e-12 * scale64).all()
    assert (np.abs(got["two_simplex"] - ref.prox("two_simplex", rows64, p=3, rhs=1.0)) <= 1e-12 * scale64).all()
    # rows on which the reference's sort-based walk stays inside its arrays
    from tests.util import two_simplex_sort_defined
    ok = two_simplex_sort_defined(ref, rows64, p=3, rhs=1.0)
    assert ok.sum() >= rows // 2
    want_s = ref.prox("two_simplex_sort", rows64[ok], p=3, rhs=1.0)
    assert (np.abs(got["two_simplex_sort"][ok] - want_s) <= 1e-12 * scale64[ok]).all()
    want_l = ref.lambert_w_exp(rows64)
    assert (np.abs(got["lambert"] - want_l) <= 1e-12 * np.maximum(1, np.abs(want_l))).all()
    r = ref.evaluate("l2_topk_hinge_smooth", X, A, labels, W=W, c=1.0, gamma=1.0, k=1)
    for i, f in enumerate(("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer",
                           "dual_regularizer")):
        assert abs(out_eval[i] - r[f]) <= 1e-12 * max(1, abs(r[f])), f
    assert abs(out_eval[6] - r["accuracy"][0]) <= 1e-12
    A_ref = np.zeros((n, m)); W_ref = np.zeros((m, d))
    rr = ref.fit("l2_topk_hinge_smooth", X, A_ref, labels, W=W_ref, c=1.0, gamma=1.0, k=1,
                 epsilon=1e-3, max_epoch=100, eval_epoch=10)
    assert int(out_fit[0]) == rr["status"] and int(out_fit[1]) == rr["epoch"]
    assert int(out_fit[2]) == len(rr["history"])
    assert abs(out_fit[3] - rr["history"][-1][0]) <= 1e-9 * max(1, abs(rr["history"][-1][0]))
    assert abs(out_fit[4] - rr["history"][-1][1]) <= 1e-9 * max(1, abs(rr["history"][-1][1]))
    assert np.abs(fit_A - A_ref).max() <= 1e-9 * max(1, np.abs(A_ref).max())
