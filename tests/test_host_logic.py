"""Host-side logic of the library that needs no GPU: the stopping rule with its time
limits, the label checks, the step from sums to a record when the device reported a
timed-out wait, and the per-device bookkeeping."""
import ctypes as C

import numpy as np

from libsdca_b200 import binding as b


def record(primal, dual):
    r = b.EvalRecord()
    r.primal = primal; r.dual = dual
    return r


def check(hostsim, status, last, before, epsilon=1e-3, epoch=1, max_epoch=100, max_cpu=0.0, cpu=0.0,
          max_wall=0.0, wall=0.0):
    f = hostsim.lib.sdcab_hostsim_check_stopping
    f.restype = C.c_int
    return f(C.c_int(status), C.byref(last) if last is not None else None,
             C.byref(before) if before is not None else None, C.c_double(epsilon), C.c_int64(epoch),
             C.c_int64(max_epoch), C.c_double(2.2e-16), C.c_double(max_cpu), C.c_double(cpu),
             C.c_double(max_wall), C.c_double(wall))


def test_stopping_rule_with_time_limits(hostsim):
    """check_stopping_criteria of the reference (include/sdca/solver/eval.h:56-109): the gap
    first, then epochs, then processor time, then wall time."""
    SOLVING, SOLVED, NO_PROGRESS, MAX_EPOCH, MAX_CPU, MAX_WALL, FAILED = 1, 2, 3, 4, 5, 6, 7
    far = record(2.0, 1.0)
    assert check(hostsim, SOLVING, far, None) == SOLVING
    assert check(hostsim, SOLVING, record(1.0005, 1.0), None) == SOLVED
    assert check(hostsim, SOLVING, record(0.9, 1.0), None) == FAILED
    assert check(hostsim, SOLVING, record(2.0, 0.5), far) == NO_PROGRESS
    assert check(hostsim, SOLVING, far, None, epoch=100) == MAX_EPOCH
    # limits of zero are no limits; a limit is reached at equality (>=)
    assert check(hostsim, SOLVING, far, None, max_cpu=0.0, cpu=1e9) == SOLVING
    assert check(hostsim, SOLVING, far, None, max_cpu=2.0, cpu=1.9) == SOLVING
    assert check(hostsim, SOLVING, far, None, max_cpu=2.0, cpu=2.0) == MAX_CPU
    assert check(hostsim, SOLVING, far, None, max_wall=3.0, wall=3.5) == MAX_WALL
    # order of the checks: epochs before cpu before wall; a solved gap before all of them
    assert check(hostsim, SOLVING, far, None, epoch=100, max_cpu=1.0, cpu=2.0) == MAX_EPOCH
    assert check(hostsim, SOLVING, far, None, max_cpu=1.0, cpu=2.0, max_wall=1.0, wall=2.0) == MAX_CPU
    assert check(hostsim, SOLVING, record(1.0005, 1.0), None, max_wall=1.0, wall=2.0) == SOLVED
    # a solver that is not running stays as it is
    assert check(hostsim, MAX_CPU, far, None) == MAX_CPU


def test_fit_stops_at_a_wall_time_limit(hostsim):
    """A fit that cannot reach its epsilon stops with max_wall_time after the epoch in
    which the limit passed (single-lane host build of the update step)."""
    rng = np.random.default_rng(5)
    n, d, m = 400, 8, 5
    X = rng.standard_normal((n, d)); labels = rng.integers(0, m, n).astype(np.int64)
    A = np.zeros((n, m)); W = np.zeros((m, d))
    obj = b.make_objective("msvm", c=1.0, k=1, from_name=hostsim.lib.sdcab_hostsim_objective_from_name)
    prob = b.make_problem(X, labels, A, W)
    crit = b.FitCriteria(0.0, 10 ** 6, 0, 0, 0, 0.0, 0.05)
    res = b.FitResult()
    evals = (b.EvalRecord * 4)()
    rc = hostsim.lib.sdcab_hostsim_fit(C.byref(obj), C.byref(prob), 1, C.byref(crit), None, evals,
                                       C.c_int64(4), C.byref(res))
    assert rc == 0
    assert b.FIT_STATUS[res.status] == "max_wall_time"
    assert res.epoch >= 1 and res.wall_seconds >= 0.05
    assert res.num_evals == 1          # the final evaluation of end_solve


def validate(hostsim, labels, offsets, n, m, ml):
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    off = np.ascontiguousarray(offsets, dtype=np.int64) if offsets is not None else None
    return hostsim.lib.sdcab_hostsim_validate_labels(
        labels.ctypes.data_as(C.c_void_p), off.ctypes.data_as(C.c_void_p) if off is not None else None,
        C.c_int64(n), C.c_int64(m), 1 if ml else 0)


def test_label_checks(hostsim):
    """include/sdca/solver/data/output.h:169-215, labels 0-based."""
    LABELS_RANGE = -5
    assert validate(hostsim, [0, 3, 2], None, 3, 4, False) == 0
    assert validate(hostsim, [0, 4, 2], None, 3, 4, False) == LABELS_RANGE
    assert validate(hostsim, [0, -1, 2], None, 3, 4, False) == LABELS_RANGE
    assert validate(hostsim, [0, 2, 1, 3], [0, 2, 4], 2, 5, True) == 0
    assert validate(hostsim, [0, 2, 1, 3], [1, 2, 4], 2, 5, True) == LABELS_RANGE      # first offset
    assert validate(hostsim, [0, 2, 1, 3], [0, 2, 2], 2, 5, True) == LABELS_RANGE      # empty example
    assert validate(hostsim, [0, 0, 1, 3], [0, 2, 4], 2, 5, True) == LABELS_RANGE      # duplicate
    assert validate(hostsim, [2, 0, 1, 3], [0, 2, 4], 2, 5, True) == LABELS_RANGE      # unsorted
    assert validate(hostsim, [0, 1, 2, 3], [0, 4], 1, 4, True) == LABELS_RANGE         # all classes
    assert validate(hostsim, [0, 5], [0, 2], 1, 5, True) == LABELS_RANGE               # out of range


def test_host_entry_points_reject_bad_labels_without_a_gpu():
    """The product library checks labels before it touches CUDA."""
    lib = b.lib()
    X = np.zeros((3, 2)); W = np.zeros((4, 2)); A = np.zeros((3, 4))
    labels = np.array([0, 9, 1], dtype=np.int64)
    obj = b.make_objective("msvm", c=1.0, k=1)
    prob = b.make_problem(X, labels, A, W)
    rec = b.EvalRecord()
    assert lib.sdcab_eval_f64(C.byref(obj), C.byref(prob), C.byref(rec), None) == -5
    crit = b.FitCriteria(1e-3, 10, 1, 0, 0, 0.0, 0.0)
    res = b.FitResult()
    assert lib.sdcab_fit_f64(C.byref(obj), C.byref(prob), C.byref(crit), None, None, C.c_int64(0),
                             C.byref(res)) == -5
    crit.max_wall_time = -1.0
    labels[1] = 2
    assert lib.sdcab_fit_f64(C.byref(obj), C.byref(prob), C.byref(crit), None, None, C.c_int64(0),
                             C.byref(res)) == -2


def test_a_timed_out_device_wait_becomes_a_status():
    """sums[6] is the device's error word: when a bounded wait inside the tensor-core
    product ran out it is non-zero and sdcab_eval_finish reports SDCAB_ERR_TIMEOUT instead
    of a record."""
    lib = b.lib()
    m = 4
    obj = b.make_objective("msvm", c=1.0, k=1)
    sums = np.zeros(8 + m); sums[5] = 10; sums[8] = 10
    rec = b.EvalRecord()
    assert lib.sdcab_eval_finish(C.byref(obj), C.c_int64(m), sums.ctypes.data_as(C.c_void_p),
                                 C.byref(rec), None) == 0
    sums[6] = 2.0
    assert lib.sdcab_eval_finish(C.byref(obj), C.c_int64(m), sums.ctypes.data_as(C.c_void_p),
                                 C.byref(rec), None) == -23
    lib.sdcab_status_string.restype = C.c_char_p
    assert lib.sdcab_status_string(-23) == b"device_wait_timeout"


def test_per_device_state_is_keyed_by_device(hostsim):
    """One process may drive several GPUs: what is set up once per device (kernel
    attributes, streams) must be set up again on the next device, not once per process."""
    order = np.array([0, 0, 1, 0, 1, 3, 3, 63, 64, -1], dtype=np.int32)
    f = hostsim.lib.sdcab_hostsim_once_per_device
    f.restype = C.c_uint64
    bits = f(order.ctypes.data_as(C.c_void_p), C.c_int(len(order)))
    first = [bool(bits >> i & 1) for i in range(len(order))]
    assert first == [True, False, True, False, False, True, False, True, False, False]


def test_test_switches_are_named():
    lib = b.lib()
    assert lib.sdcab_test_set(b"eval_chunk", C.c_int64(0)) == 0
    assert lib.sdcab_test_set(b"gemm_simt", C.c_int64(0)) == 0
    assert lib.sdcab_test_set(b"no_such_switch", C.c_int64(1)) == -1
