"""Build recipe for the CPU oracle (test infrastructure, never a product path).

Two libraries are produced:

* ``oracle/libsdca_oracle.so`` -- the C restatement in ``sdca_oracle.c`` (always
  built; needs only gcc).
* ``oracle/_ref/libsdca_ref.so`` -- ``ref_shim.cpp`` compiled against the
  reference's own, unmodified header tree.  Built only where that tree is
  present (``SDCA_REFERENCE_DIR``, or a ``reference`` folder beside this repository);
  elsewhere the prebuilt file that travelled with the repository is used as it is.
  A second build of the same shim with ``-DSDCA_ACCURATE_MATH`` goes to
  ``oracle/_ref/libsdca_ref_accurate.so``.

The reference flags follow its default (non ``SDCA_ACCURATE_MATH``) build, but
without ``-Ofast``/``-ffast-math`` so that results do not depend on the
compiler's reassociation: ``-std=c++14 -O2 -include limits``.  ``-include
limits`` is needed because ``include/sdca/math/log_exp.h`` of the reference uses
``std::numeric_limits`` without including ``<limits>``.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference's source tree: named by the environment, else looked for beside this
# repository (../reference); where neither exists the prebuilt library is used
REF_DIR = os.environ.get("SDCA_REFERENCE_DIR") or os.path.normpath(os.path.join(HERE, "..", "..", "reference"))
REF_SO = os.path.join(HERE, "_ref", "libsdca_ref.so")
# the same shim against the same headers with SDCA_ACCURATE_MATH defined: the reference's
# optional exact recomputation of t (prox/knapsack_eq.h:87-106) and of W (eval/core.h:148-182)
REF_ACCURATE_SO = os.path.join(HERE, "_ref", "libsdca_ref_accurate.so")
ORACLE_SO = os.path.join(HERE, "libsdca_oracle.so")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("command failed: " + " ".join(cmd))


def build_restatement(force=False):
    src = [os.path.join(HERE, "sdca_oracle.c")]
    inc = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".inc") or f.endswith(".h")]
    if not os.path.exists(src[0]):
        return None
    if force or not _newer(ORACLE_SO, src + inc):
        _run(["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-fno-fast-math", "-o", ORACLE_SO]
             + src + ["-lm", "-lpthread"])
    return ORACLE_SO


def build_reference(force=False):
    """Compile the reference headers where they lie; returns the .so path or None."""
    inc = os.path.join(REF_DIR, "include")
    shim = os.path.join(HERE, "ref_shim.cpp")
    blas = os.path.join(HERE, "cblas_seq.c")
    if not os.path.isdir(inc):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, [shim, blas]) and _newer(REF_ACCURATE_SO, [shim, blas]):
        return REF_SO
    os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
    obj = os.path.join(HERE, "_ref", "cblas_seq.o")
    _run(["gcc", "-std=c11", "-O2", "-fPIC", "-fno-fast-math", "-c", blas, "-o", obj])
    _run(["g++", "-std=c++14", "-O2", "-fPIC", "-shared", "-include", "limits",
          "-DBLAS_DEFAULT_LOCAL_HEADER", "-I", inc, shim, obj, "-o", REF_SO,
          "-lpthread", "-ldl"])
    _run(["g++", "-std=c++14", "-O2", "-fPIC", "-shared", "-include", "limits",
          "-DBLAS_DEFAULT_LOCAL_HEADER", "-DSDCA_ACCURATE_MATH", "-I", inc, shim, obj, "-o",
          REF_ACCURATE_SO, "-lpthread", "-ldl"])
    return REF_SO


def build_all(force=False):
    return build_restatement(force), build_reference(force)


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
