"""Shared parity metrics for the tests."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def split_prefix(d, prefix):
    return {k[len(prefix):]: v for k, v in d.items() if k.startswith(prefix)}


def max_abs_rel(a, ref):
    """max|a - ref| / max|ref| for one tensor."""
    den = float(np.abs(ref).max())
    return float(np.abs(a.astype(np.float64) - ref.astype(np.float64)).max()) / (den if den > 0 else 1.0)


def assert_grads_close(got, ref, tol=1e-4, floor_rel=1e-6):
    """Every parameter gradient within tol (max-abs-rel).  Tensors whose reference magnitude is below
    floor_rel x the largest gradient magnitude in the model are analytically zero (the key-projection
    bias: softmax is shift invariant) and hold rounding noise on both sides; they are compared
    absolutely against that floor instead."""
    assert set(got) == set(ref), (sorted(set(got) ^ set(ref)))
    biggest = max(float(np.abs(v).max()) for v in ref.values())
    floor = floor_rel * biggest
    worst = ("", 0.0)
    for k in ref:
        assert got[k].shape == ref[k].shape, k
        if float(np.abs(ref[k]).max()) < floor:
            assert float(np.abs(got[k]).max()) < 10 * floor, (k, float(np.abs(got[k]).max()), floor)
            continue
        e = max_abs_rel(got[k], ref[k])
        if e > worst[1]:
            worst = (k, e)
        assert e <= tol, (k, e)
    return worst
