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


def assert_matches_digest(got, gold, prefix, tol=1e-4, floor_rel=1e-6, abs_tol=None):
    """The same bar as assert_grads_close against a digest fixture (tests/golden/make_golden.py: digest): the fixed strided
    sample of every tensor within tol of the reference relative to the reference tensor's max |x| (or within abs_tol when
    given), and the tensor's sum of squares within 2 * tol, which covers the elements the sample leaves out."""
    from tests.golden.make_golden import DIGEST_STRIDE

    stats = split_prefix(gold, "stat/" + prefix)
    samples = split_prefix(gold, "sample/" + prefix)
    assert set(got) == set(stats), sorted(set(got) ^ set(stats))
    biggest = max(float(s[2]) for s in stats.values())
    floor = floor_rel * biggest
    worst = ("", 0.0)
    for k, (s_sum, s_sq, s_max) in stats.items():
        flat = got[k].reshape(-1)
        assert flat[::DIGEST_STRIDE].shape == samples[k].shape, k
        if s_max < floor:  # analytically zero (key-projection bias): rounding noise on both sides
            assert float(np.abs(flat).max()) < 10 * floor, (k, float(np.abs(flat).max()), floor)
            continue
        diff = float(np.abs(flat[::DIGEST_STRIDE].astype(np.float64) - samples[k].astype(np.float64)).max())
        if abs_tol is not None:
            assert diff < abs_tol, (k, diff)
        else:
            e = diff / s_max
            if e > worst[1]:
                worst = (k, e)
            assert e <= tol, (k, e)
        sq = float((flat.astype(np.float64) ** 2).sum())
        assert abs(sq - s_sq) <= 2 * (tol if abs_tol is None else 1e-3) * s_sq, (k, sq, s_sq)
    return worst
