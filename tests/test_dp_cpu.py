"""Data-parallel bucket bookkeeping on CPU: the C++ ParamArena logic is replayed without a GPU (gct_dp_simulate) and its
recorded bucket reductions drive a host all-reduce — in-process for the ordering rules, and over gloo with two ranks for the
exchange itself."""
import ctypes
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def simulate(sizes, bucket_elems, world, accum_hint, accum, steps):
    import __graft_entry__ as entry

    entry.build()
    from gradcraft_b200 import trainer

    L = trainer._lib()
    L.gct_dp_simulate.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                                  ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
    s = np.asarray(sizes, dtype=np.int64)
    ev = np.zeros((4096, 6), dtype=np.int64)
    n, total = ctypes.c_int64(), ctypes.c_int64()
    rc = L.gct_dp_simulate(s.ctypes.data, len(s), bucket_elems, world, accum_hint, accum, steps, ev.ctypes.data, len(ev), ctypes.byref(n), ctypes.byref(total))
    assert rc == 0, L.gct_last_error()
    return ev[: n.value], total.value


SIZES = [1024, 1024, 5000, 300000, 300000, 70, 1024 * 1024, 64, 2048 * 64, 96 * 1024]


def test_buckets_partition_the_arena_and_fire_in_finality_order():
    ev, total = simulate(SIZES, 256 * 1024, world=2, accum_hint=2, accum=2, steps=3)
    per_step = {}
    for step, mb, slot, bucket, begin, count in ev:
        per_step.setdefault(step, []).append((mb, slot, bucket, begin, count))
    assert sorted(per_step) == [0, 1, 2]
    for step, rows in per_step.items():
        # nothing is reduced before the last micro-batch: earlier gradients are still accumulating
        assert all(mb >= 1 for mb, *_ in rows)
        buckets = [r[2] for r in rows]
        assert buckets == sorted(buckets) and len(set(buckets)) == len(buckets)
        covered = 0
        for mb, slot, bucket, begin, count in rows:
            assert begin == covered  # contiguous, in arena order
            covered += count
        assert covered == total
        # every bucket but possibly the last fired inside the sweep (overlapped), right after its last slot became final
        overlapped = [r for r in rows if r[1] >= 0]
        assert len(overlapped) >= len(rows) - 1
        slots = [r[1] for r in overlapped]
        assert slots == sorted(slots)
    assert total % 1024 == 0 and total >= sum(SIZES)


def test_accumulation_count_is_learnt_on_the_first_step():
    ev, total = simulate(SIZES, 256 * 1024, world=2, accum_hint=0, accum=3, steps=2)
    first = [r for r in ev if r[0] == 0]
    later = [r for r in ev if r[0] == 1]
    assert all(r[2] == -1 for r in first)  # unknown count: everything reduced when the optimizer asks for the gradients
    assert any(r[2] >= 0 and r[1] == 2 for r in later)  # afterwards the third (last) backward overlaps its buckets
    assert sum(r[5] for r in first) == total == sum(r[5] for r in later)


def test_single_rank_never_reduces():
    ev, _ = simulate(SIZES, 256 * 1024, world=1, accum_hint=1, accum=1, steps=2)
    assert len(ev) == 0


def _rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    ev, total = simulate(SIZES, 256 * 1024, world=world, accum_hint=1, accum=1, steps=1)
    g = torch.from_numpy(np.random.default_rng(10 + rank).standard_normal(total).astype(np.float32))
    whole = g.clone()
    for step, mb, slot, bucket, begin, count in ev:  # the host all-reduce stand-in, bucket by bucket, in firing order
        part = g[begin : begin + count]
        dist.all_reduce(part)
        part /= world
    dist.all_reduce(whole)
    whole /= world
    q.put((rank, bool(torch.equal(g, whole)), float(g.double().sum())))
    dist.destroy_process_group()


def test_two_ranks_bucketed_average_equals_whole_average_gloo():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 300)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in out)
    assert out[0][2] == out[1][2]  # both ranks hold identical reduced gradients


# ---- failure path of the gradient exchange, host side only (no GPU is made to fail) ------------------------------------------
def _lib():
    import __graft_entry__ as entry

    entry.build()
    from gradcraft_b200 import capi

    return capi, capi.lib()


@pytest.mark.parametrize("scenario,status,aborts", [(0, "OK", 0), (1, "TIMEOUT", 1), (2, "NCCL_ERROR", 1), (3, "TIMEOUT", 0), (4, "NCCL_ERROR", 0)])
def test_communicator_watchdog_and_guarded_creation(scenario, status, aborts):
    """The watchdog and the creation timeout that guard the NCCL communicator, driven by stand-ins for the NCCL calls: a
    healthy reduction, one that never completes, an asynchronous error, a creation that never returns (a peer never joined)
    and one that fails (bad unique id).  Failures end in a status code and one ncclCommAbort, never in a wait without end."""
    capi, lib = _lib()
    n = ctypes.c_int(-1)
    if status == "OK":
        assert lib.dp_selftest(scenario, 150, ctypes.byref(n)) == capi.OK
    else:
        with pytest.raises(capi.GcbError) as e:
            lib.dp_selftest(scenario, 150, ctypes.byref(n))
        assert e.value.status == getattr(capi, status)
    assert n.value == aborts


def _rendezvous_rank(rank, world, port, directory, joins, q):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    capi, lib = _lib()
    status = "skipped"
    if joins:
        try:
            lib.dp_selftest_rendezvous(directory.encode(), rank, world, 1500)
            status = "OK"
        except capi.GcbError as e:
            status = {capi.TIMEOUT: "TIMEOUT", capi.NCCL_ERROR: "NCCL_ERROR"}.get(e.status, str(e.status))
    # the survivors learn on the host who made it (a store / heartbeat in a real job) before anything is queued on a device
    seen = [None] * world
    dist.all_gather_object(seen, status)
    q.put((rank, status, seen))
    dist.destroy_process_group()


@pytest.mark.parametrize("case", ["all_join", "one_never_joins", "wrong_id"])
def test_two_ranks_rendezvous_under_the_creation_timeout_gloo(case, tmp_path):
    """Two CPU ranks (gloo for the out-of-band channel) go through the guarded communicator creation with a directory
    rendezvous standing in for ncclCommInitRank: both join -> OK; rank 1 never calls it -> rank 0 gets GCB_TIMEOUT instead of
    waiting for ever, before any collective exists; a directory that does not exist (wrong id) -> GCB_NCCL_ERROR at once."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 90) + {"all_join": 0, "one_never_joins": 100, "wrong_id": 200}[case]
    directory = str(tmp_path / ("absent" if case == "wrong_id" else ""))
    procs = [ctx.Process(target=_rendezvous_rank, args=(r, 2, port, directory, not (case == "one_never_joins" and r == 1), q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = {"all_join": ["OK", "OK"], "one_never_joins": ["TIMEOUT", "skipped"], "wrong_id": ["NCCL_ERROR", "NCCL_ERROR"]}[case]
    assert [s for _, s, _ in out] == want
    assert all(seen == want for _, _, seen in out)  # every rank knows the outcome of every other
