"""The microbenchmark shapes and the full 180M-parameter training step, checked through properties that do not need a
CPU run of that size: conservation laws of each backward formula, agreement with the numpy oracle on a strided sample of
rows, run-to-run bit identity, and the accumulation identity of the training step.  Everything goes through the C ABI."""
import numpy as np
import pytest

from oracle import numpy_oracle as O
from oracle import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    from gradcraft_b200 import capi

    ctx = capi.Context(0)
    yield ctx, torch, capi
    ctx.sync()
    ctx.close()
    torch.cuda.empty_cache()


def test_softmax_ce_backward_16384_x_32768(env):
    """dlogits = (p - onehot) * upstream / rows: every row sums to zero, the target entry is the only negative one, and a
    sample of rows equals the oracle; written in place over the probabilities."""
    ctx, torch, capi = env
    M, V = 16384, 32768
    torch.manual_seed(0)
    logits = torch.randn(M, V, device="cuda") * 3
    tg = torch.randint(0, V, (M,), dtype=torch.int32, device="cuda")
    loss = torch.empty(1, device="cuda")
    ctx.softmax_ce_fwd_f32(loss, logits, logits, tg, capi.IDX_I32, M, V, 1e-5)  # probabilities over the logits
    rows = [0, 1, 777, 8191, 16383]
    p_rows = logits[rows].cpu().numpy()
    ctx.softmax_ce_bwd_f32(logits, logits, tg, capi.IDX_I32, 0.5, M, V, 0)      # gradient over the probabilities
    ctx.sync()
    assert float(logits.double().sum(1).abs().max()) < 1e-9
    neg = (logits < 0).sum(1)
    assert int(neg.min()) == 1 and int(neg.max()) == 1
    assert bool((logits.gather(1, tg.long()[:, None]) < 0).all())
    t_host = tg.cpu().numpy()
    for i, r in enumerate(rows):
        ref = O.softmax_ce_bwd(p_rows[i:i + 1], t_host[r:r + 1].astype(np.int64), np.float32(0.5)) * (1.0 / M)
        got = logits[r].cpu().numpy()
        assert float(np.abs(got - ref[0]).max()) <= 1e-6 * float(np.abs(ref).max()) + 1e-12
    del logits


def test_layernorm_backward_16384_x_1024(env):
    """dx of every row is orthogonal to the constant vector and to the normalised row (the two directions LayerNorm
    removes); dgamma / dbeta equal float64 column sums; a sample of rows equals the oracle; two runs are bit-identical."""
    ctx, torch, capi = env
    M, C = 16384, 1024
    torch.manual_seed(1)
    x, dy = torch.randn(M, C, device="cuda") * 2 + 0.3, torch.randn(M, C, device="cuda") * 1e-2
    g, b = torch.rand(C, device="cuda") + 0.5, torch.zeros(C, device="cuda")
    y, mu, rs = torch.empty_like(x), torch.empty(M, device="cuda"), torch.empty(M, device="cuda")
    ctx.layernorm_fwd_f32(y, mu, rs, x, g, b, M, C, 1e-5)
    outs = []
    for _ in range(2):
        dx, dg, db = torch.empty_like(x), torch.empty(C, device="cuda"), torch.empty(C, device="cuda")
        ctx.layernorm_bwd_f32(dx, dg, db, dy, x, g, mu, rs, M, C, 0, 0)
        ctx.sync()
        outs.append((dx, dg, db))
    assert all(torch.equal(a, b_) for a, b_ in zip(*outs))
    dx, dg, db = outs[0]
    xhat = ((x - mu[:, None]) * rs[:, None]).double()
    scale = float(dx.abs().max()) * C
    assert float(dx.double().sum(1).abs().max()) < 1e-5 * scale
    assert float((dx.double() * xhat).sum(1).abs().max()) < 1e-5 * scale
    ref_db, ref_dg = dy.double().sum(0), (dy.double() * xhat).sum(0)
    assert float((db.double() - ref_db).abs().max() / ref_db.abs().max()) < 1e-5
    assert float((dg.double() - ref_dg).abs().max() / ref_dg.abs().max()) < 1e-5
    rows = [0, 5, 4735, 4736, 16383]
    rdx, _, _ = O.layernorm_bwd(dy[rows].cpu().numpy(), x[rows].cpu().numpy(), g.cpu().numpy(), mu[rows].cpu().numpy(), rs[rows].cpu().numpy())
    assert float(np.abs(dx[rows].cpu().numpy() - rdx).max() / np.abs(rdx).max()) < 1e-5


def test_gelu_backward_16384_x_4096_sample(env):
    ctx, torch, capi = env
    M, F = 16384, 4096
    torch.manual_seed(2)
    x, dy = torch.randn(M, F, device="cuda") * 2, torch.randn(M, F, device="cuda") * 1e-2
    dx = torch.empty_like(x)
    ctx.gelu_bwd_f32(dx, dy, x, M * F, 0)
    ctx.sync()
    flat = slice(0, M * F, 9973)  # a fixed stride through the whole tensor
    ref = O.gelu_bwd(dy.reshape(-1)[flat].cpu().numpy(), x.reshape(-1)[flat].cpu().numpy())
    got = dx.reshape(-1)[flat].cpu().numpy()
    assert float(np.abs(got - ref).max() / np.abs(ref).max()) < 1e-5
    ctx.gelu_bwd_f32(dx, dy, x, M * F, 1)  # accumulate form doubles it
    ctx.sync()
    assert float(np.abs(dx.reshape(-1)[flat].cpu().numpy() - 2 * ref).max() / np.abs(ref).max()) < 2e-5


def test_causal_softmax_backward_16_x_16_x_1024_x_1024(env):
    """dS = scale * P * (dP - sum_j dP P): every row sums to zero, nothing above the diagonal, a sample of rows equals the oracle."""
    ctx, torch, capi = env
    Bn, H, T = 16, 16, 1024
    rows = Bn * H * T
    torch.manual_seed(3)
    S = torch.randn(rows, T, device="cuda") * 2
    ctx.causal_softmax_fwd_f32(S, S, 0.125, rows, T)
    dP = torch.randn(rows, T, device="cuda") * 1e-2
    pick = [0, 1, 1023, 1024 * 7 + 511, rows - 1]
    p_rows, dp_rows = S[pick].cpu().numpy(), dP[pick].cpu().numpy()
    ctx.causal_softmax_bwd_f32(dP, dP, S, 0.125, rows, T, 0)
    ctx.sync()
    assert float(dP.double().sum(1).abs().max()) < 1e-7
    i = torch.arange(rows, device="cuda") % T
    above = torch.arange(T, device="cuda")[None, :] > i[:, None]
    assert bool((dP[above] == 0).all())
    for k, r in enumerate(pick):
        p, d = p_rows[k].astype(np.float64), dp_rows[k].astype(np.float64)
        ref = 0.125 * p * (d - (d * p).sum())
        assert float(np.abs(dP[r].cpu().numpy() - ref).max()) <= 1e-5 * float(np.abs(ref).max()) + 1e-12
    del S, dP, above


def test_full_size_training_step_properties():
    """The 180M-parameter model at the benchmark's batch (32 sequences of 1024 tokens): the first loss sits near ln(vocab)
    for N(0, 0.02) weights; the clipper's norm equals the norm of the downloaded gradients; the step is bit-identical from
    run to run (sorted scatter-add, ordered K slices, ordered bias sums); and the same batch fed as two micro-batches of
    weight 1/2 accumulates to the one-micro-batch gradients (the beta = 1 paths of every GEMM and kernel at full size)."""
    import torch

    from gradcraft_b200.trainer import Trainer

    arch, V, T, C, H, L, F, B = "lngelu", 32768, 1024, 1024, 16, 12, 4096, 32
    w = synth.gpt_weights(arch, V, T, C, H, L, F, seed=0)
    X, Y = (np.ascontiguousarray(a) for a in synth.token_batches(1000, 1, B, T, V)[0])
    tr = Trainer(arch, V, T, C, H, L, F, clip=1.0)
    try:
        tr.load(w)

        def grads_of(accum):
            tr.zero_grad()
            loss = 0.0
            for _ in range(accum):
                loss += tr.forward_backward(X, Y, accum)
            return loss, tr.get("grad")

        loss1, g1 = grads_of(1)
        assert abs(loss1 - np.log(V)) < 0.5, loss1  # near-uniform predictions (the tied head and Zipf targets shift it a little)
        assert all(np.isfinite(g).all() for g in g1.values())
        loss1b, g1b = grads_of(1)
        assert loss1b == loss1 and all(np.array_equal(g1[k], g1b[k]) for k in g1)
        loss2, g2 = grads_of(2)
        assert abs(loss2 - loss1) < 1e-5 * loss1
        big = max(float(np.abs(g).max()) for g in g1.values())
        for k in g1:
            ref_max = float(np.abs(g1[k]).max())
            if ref_max < 1e-6 * big:
                continue  # analytically zero tensors hold rounding noise
            assert float(np.abs(g2[k] - g1[k]).max()) <= 2e-5 * ref_max, k
        exact = float(np.sqrt(sum(float((g.astype(np.float64) ** 2).sum()) for g in g2.values())))
        norm = tr.optimizer_step(want_norm=True)
        assert abs(norm - exact) / exact < 1e-5, (norm, exact)
        after = tr.get("param")
        assert all(np.isfinite(a).all() for a in after.values())
        moved = max(float(np.abs(after[k] - w[k].reshape(-1)).max()) for k in after)
        assert 0 < moved <= 3.5e-4  # one AdamW step moves a weight by at most lr (plus decay)
    finally:
        tr.close()
        torch.cuda.empty_cache()
