"""sdca_b200: B200 (sm_100a) kernels for libsdca's batched proximal operators and
duality-gap evaluation, behind a C ABI (``include/sdca_b200.h``).

This package is a thin ctypes binding used by the tests and the benchmark; the
product is the shared library ``libsdca_b200/libsdca_b200.so``.  There is no CPU
fallback: importing works without a GPU (so that symbols can be inspected), but
every compute call needs a CUDA device and raises ``SdcabError`` otherwise.
"""
from .binding import (  # noqa: F401
    SdcabError,
    ProxOpts,
    Thresholds,
    lib,
    library_path,
    prox,
    prox_,
    prox_to,
    thresholds,
    lambert_w_exp_,
    status_string,
    PROX_NAMES,
    evaluate,
    eval_sums_,
    eval_finish,
    make_objective,
    make_problem,
    fit_,
    epoch_permutations,
    primal_from_dual,
    train,
)
