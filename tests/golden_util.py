"""Loaders of the committed golden vectors (tests/golden/*.npz, produced by
tests/golden/make_golden.py from the reference's own headers)."""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def prox_cases():
    z = np.load(os.path.join(HERE, "golden", "prox_golden.npz"))
    keys = sorted({k.split("_")[0] for k in z.files})
    for key in keys:
        o = z[key + "_opts"]
        name = str(z[key + "_name"])
        kw = dict(lo=o[0], hi=o[1], rhs=o[2], rho=o[3], alpha=o[4], k=int(o[5]), p=int(o[6]))
        thr = z[key + "_thr"] if key + "_thr" in z.files else None
        yield name, z[key + "_in"], kw, z[key + "_out"], thr


def eval_cases():
    z = np.load(os.path.join(HERE, "golden", "eval_golden.npz"))
    keys = sorted({k.split("_")[0] for k in z.files})
    for key in keys:
        offsets = z[key + "_offsets"]
        yield dict(objective=str(z[key + "_objective"]), kernel=bool(z[key + "_kernel"]),
                   data=z[key + "_data"], A=z[key + "_A"], W=z[key + "_W"],
                   labels=z[key + "_labels"], offsets=offsets if len(offsets) else None,
                   c=float(z[key + "_params"][0]), gamma=float(z[key + "_params"][1]),
                   k=int(z[key + "_params"][2]), record=z[key + "_record"],
                   accuracy=z[key + "_accuracy"])


def fit_cases():
    z = np.load(os.path.join(HERE, "golden", "fit_golden.npz"))
    keys = sorted({k.split("_")[0] for k in z.files if k.startswith("fit")})
    for key in keys:
        prm = z[key + "_params"]
        offsets = z[key + "_offsets"]
        yield dict(objective=str(z[key + "_objective"]), kernel=bool(z[key + "_kernel"]),
                   offsets=offsets if len(offsets) else None,
                   data=z[key + "_data"], labels=z[key + "_labels"], c=float(prm[0]),
                   gamma=float(prm[1]), k=int(prm[2]), epsilon=float(prm[3]), max_epoch=int(prm[4]),
                   eval_epoch=int(prm[5]), A=z[key + "_A"], W=z[key + "_W"],
                   history=z[key + "_history"], status=int(z[key + "_status"][0]),
                   epoch=int(z[key + "_status"][1]))


def epoch_orders():
    z = np.load(os.path.join(HERE, "golden", "fit_golden.npz"))
    return z["order_n50000_first64"], z["order_n1000"]
