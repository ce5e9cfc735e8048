"""The reference's train.cpp, compiled unchanged against this repository's host API and linked with the sm_100a backend
(built by __graft_entry__.build() wherever the reference tree is present), trains a small model on a synthetic token file."""
import csv
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_reference_train_cpp_runs_on_the_new_backend(tmp_path):
    from gradcraft_b200 import build, synth

    binary = build.build_reference_train()
    if binary is None or not os.path.exists(binary):
        pytest.skip("train_ref was not built (no reference tree where the library was built)")
    V, T = 512, 64
    tokens = synth.zipf_tokens(3, 40 * (T + 1) * 8, V).astype("<u4")  # dataset.bin format: little-endian uint32 tokens
    data = tmp_path / "dataset.bin"
    tokens.tofile(data)
    out = tmp_path / "model"
    cmd = [binary, "--dataset", str(data), "--model_dir", str(out), "--steps", "8", "--vocab_size", str(V), "--seq_len", str(T), "--embed_dim", "128", "--num_heads", "4",
           "--num_layers", "2", "--batch_size", "4", "--target_batch", "8", "--print_every", "1", "--checkpoint_every", "4", "--max_lr", "3e-3", "--min_lr", "3e-4"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rows = list(csv.DictReader(open(out / "training_log.csv")))
    losses = [float(x["loss"]) for x in rows]
    assert len(losses) == 8 and all(np.isfinite(losses))
    assert abs(losses[0] - np.log(V)) < 0.5  # fresh N(0, 0.02) weights: near-uniform predictions
    assert losses[-1] < losses[0]            # and it learns
    assert all(float(x["norm"]) > 0 for x in rows)
    for f in ("trained_model.bin", "latest_model.bin", "latest_optim.bin", "latest_scheduler.bin", "config.bin"):
        assert (out / f).exists(), f
    # resume from the checkpoint it wrote
    resumed = [a if a != "8" or cmd[i - 1] != "--steps" else "10" for i, a in enumerate(cmd)] + ["--resume"]
    r2 = subprocess.run(resumed, capture_output=True, text=True, timeout=300)
    assert r2.returncode == 0, r2.stdout[-2000:] + r2.stderr[-2000:]
    # the checkpoint of step 4 was written after the scheduler had advanced to t = 5, which is where the loop restarts
    assert "Successfully resumed state from step: 5" in r2.stdout
    rows2 = list(csv.DictReader(open(out / "training_log.csv")))
    assert [int(x["step"]) for x in rows2[8:]] == [5, 6, 7, 8, 9]
    assert float(rows2[-1]["loss"]) < losses[0]
