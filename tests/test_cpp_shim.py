"""The header-only C++ shim (include/sdca_b200.hpp) compiles against the C ABI
with the reference's call shapes (no GPU is needed to compile and link)."""
import os
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SOURCE = r'''
#include <vector>
#include "sdca_b200.hpp"
int main(int argc, char**) {
  std::vector<float> a(8 * 4, 1.0f), aux(8);
  std::vector<double> b(8 * 4, 1.0);
  if (argc > 100) {  // never executed here: this test only compiles and links
    sdca::b200::prox_topk_simplex(8, a.data(), a.data() + a.size(), aux.data(), 3, 1.0);
    sdca::b200::prox_topk_cone<float>(8, a.data(), a.data() + a.size(), aux.data(), 3);
    sdca::b200::prox_knapsack_eq(8, b.data(), b.data() + b.size(), b.data());
    sdca::b200::prox_two_simplex(8, 3, b.data(), b.data() + b.size(), b.data(), 1.0);
    sdca::b200::apply_lambert_w_exp(8, a.data(), a.data() + a.size());
    sdcab_objective o; sdcab_objective_from_name("msvm_smooth", 1.0, 1.0, 1, &o);
    sdcab_problem p = sdcab_problem();
    sdca::b200::evaluate_dataset<float>(o, p);
    sdcab_fit_criteria c = {1e-3, 100, 10, 0, 0};
    std::vector<sdcab_eval_record> evals;
    sdcab_fit_result r = sdca::b200::solve<double>(o, p, c, &evals);
    (void)r;
  }
  return 0;
}
'''


def test_shim_compiles_and_links():
    import libsdca_b200
    lib = libsdca_b200.library_path()
    if not os.path.exists(lib):
        pytest.skip("library not built")
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "shim.cpp")
        open(src, "w").write(SOURCE)
        exe = os.path.join(tmp, "shim")
        cmd = ["g++", "-std=c++11", "-I", os.path.join(ROOT, "include"), src, "-o", exe, lib,
               "-Wl,-rpath," + os.path.dirname(lib), "-Wl,-rpath,/usr/local/cuda/lib64"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
