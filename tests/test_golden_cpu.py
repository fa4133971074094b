"""The committed golden vectors (outputs of the reference itself) against the
C restatement and against the host-lane build of the CUDA threshold code."""
import numpy as np
import pytest

from tests.golden_util import eval_cases, prox_cases
from tests.util import scaled_error, tolerance


@pytest.fixture(scope="module")
def port():
    from oracle import build_oracle, refapi
    build_oracle.build_restatement()
    return refapi.restatement()


def test_restatement_reproduces_golden_prox(port):
    n = 0
    for name, a, kw, out, thr in prox_cases():
        x = port.prox(name, a, **kw)
        assert scaled_error(x, out, a).max() <= tolerance(a.dtype, "double", a.shape[1]), name
        n += 1
    assert n >= 70


def test_hostsim_reproduces_golden_prox(hostsim):
    for name, a, kw, out, thr in prox_cases():
        x, _ = hostsim.run(name, a, **kw)
        assert scaled_error(x, out, a).max() <= tolerance(a.dtype, "double", a.shape[1]), name


def test_restatement_reproduces_golden_eval(port):
    from oracle.refapi import EVAL_FIELDS
    n = 0
    for c in eval_cases():
        kw = dict(c=c["c"], gamma=c["gamma"], k=c["k"], offsets=c["offsets"])
        if c["kernel"]:
            rec = port.evaluate(c["objective"], c["data"], c["A"].copy(), c["labels"], kernel=True, **kw)
        else:
            rec = port.evaluate(c["objective"], c["data"], c["A"].copy(), c["labels"], W=c["W"], **kw)
        tol = 1e-12 if c["data"].dtype == np.float64 else 1e-5
        for i, f in enumerate(EVAL_FIELDS):
            assert abs(rec[f] - c["record"][i]) <= tol * max(1, abs(c["record"][i])), (c["objective"], f)
        assert np.allclose(rec["accuracy"], c["accuracy"], atol=1e-12)
        n += 1
    assert n == 36
