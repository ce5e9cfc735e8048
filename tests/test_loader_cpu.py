"""gradc::DataLoader of this repository (prefetch thread + recycled host blocks) hands out exactly the batches of the
reference's DataLoader, in the same order: against the order recorded from the compiled reference
(tests/golden/loader_order.txt, written by tests/golden/make_golden.py), with and without the prefetch thread, and
across a change of batch size while batches are already prepared ahead."""
import os
import subprocess

import pytest

from tests.golden.make_golden import LOADER_CASES, loader_dataset

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def checker(tmp_path_factory):
    from gradcraft_b200 import build

    build.build()
    exe = str(tmp_path_factory.mktemp("loader") / "loader_check")
    pkg = os.path.join(ROOT, "gradcraft_b200")
    cmd = ["g++", "-std=c++23", "-O1", "-I", pkg, "-I/usr/local/cuda/include", os.path.join(ROOT, "tests", "loader_check.cpp"), "-o", exe, "-L" + pkg, "-lgradc_b200",
           "-L/usr/local/cuda/lib64", "-lcudart", "-pthread", "-Wl,-rpath," + pkg, "-Wl,-rpath,/usr/local/cuda/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


def golden():
    out, name = {}, None
    for line in open(os.path.join(ROOT, "tests", "golden", "loader_order.txt")):
        line = line.strip()
        if line.startswith("#"):
            name = line[1:].strip()
            out[name] = []
        elif line:
            out[name].append(line)
    return out


@pytest.mark.parametrize("case", list(LOADER_CASES))
@pytest.mark.parametrize("prefetch", ["2", "0", "5"])
def test_batches_equal_the_reference_loader(checker, tmp_path, case, prefetch):
    seed, n_tok, vocab, T, n, b1, b2, sw = LOADER_CASES[case]
    path = str(tmp_path / "dataset.bin")
    loader_dataset(path, seed, n_tok, vocab)
    env = dict(os.environ, GRADC_LOADER_PINNED="0", GRADC_LOADER_PREFETCH=prefetch)  # pageable blocks: no GPU on this machine
    r = subprocess.run([checker, path, str(T), str(n), str(b1), str(b2), str(sw)], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip().splitlines() == golden()[case]
