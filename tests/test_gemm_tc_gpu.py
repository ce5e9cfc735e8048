"""The tcgen05 split-fp32 GEMM engine against float64 numpy: every operand layout, tile width, ragged edges, bias / beta
epilogues, head-strided batches and split-K.  Tolerance: max-abs-rel 2e-5 per output (fp32-class accuracy; plain TF32
would sit near 1e-3)."""
import os

import numpy as np
import pytest

from tests.helpers import max_abs_rel

pytestmark = pytest.mark.gpu
TOL = 2e-5


@pytest.fixture(scope="module")
def env():
    import torch

    from gradcraft_b200 import capi

    ctx = capi.Context(0)
    ctx.ctx_set_gemm_engine(2)
    yield ctx, torch, capi
    ctx.ctx_set_gemm_engine(0)
    ctx.sync()
    ctx.close()


def rnd(seed, *shape):
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)


@pytest.mark.parametrize("opa,opb,M,N,K", [
    (0, 1, 128, 64, 64), (0, 0, 128, 256, 32), (1, 0, 128, 128, 48), (1, 1, 128, 128, 16),
    (0, 0, 300, 520, 100), (0, 1, 257, 1000, 132), (1, 0, 200, 72, 1028), (1, 1, 132, 260, 36),
    (0, 0, 1024, 1024, 1024), (1, 0, 512, 512, 8192),
    (0, 0, 300, 64, 1000), (1, 0, 260, 48, 520), (0, 1, 640, 64, 4096), (1, 1, 384, 36, 272),  # 64-wide tiles with long K loops, ragged edges
])
def test_tc_gemm_vs_numpy(env, opa, opb, M, N, K):
    ctx, torch, capi = env
    A = rnd(1, *((K, M) if opa else (M, K)))
    B = rnd(2, *((N, K) if opb else (K, N)))
    C0, bias = rnd(3, M, N), rnd(4, N)
    dA, dB, dbias = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), torch.from_numpy(bias).cuda()
    a = (A.T if opa else A).astype(np.float64)
    b = (B.T if opb else B).astype(np.float64)
    C = torch.from_numpy(C0).cuda()
    ctx.gemm_f32(opa, opb, M, N, K, 1.0, dA, A.shape[1], dB, B.shape[1], 0.0, C, N, None)
    ctx.sync()
    assert ctx.ctx_last_gemm_engine() == 2
    assert max_abs_rel(C.cpu().numpy(), a @ b) < TOL
    C = torch.from_numpy(C0).cuda()
    ctx.gemm_f32(opa, opb, M, N, K, 0.5, dA, A.shape[1], dB, B.shape[1], 1.0, C, N, dbias)
    ctx.sync()
    assert max_abs_rel(C.cpu().numpy(), 0.5 * (a @ b) + C0 + bias) < TOL


@pytest.mark.parametrize("mode", [2, 1, 0])
def test_tc_gemm_is_fp32_class_not_tf32_class(env, mode):
    """Operands 1 + 1e-3 z: rounding them to TF32 once would cost ~4e-5 of the result here; every split mode must stay an
    order of magnitude below that.  (The residual error is the tensor core's truncating fp32 accumulation: a bias of a few
    1e-6 on all-positive sums, measured 5e-6 at K = 256 and 2e-5 at K = 32768, the same for the TF32 + 2 x BF16 split and
    for three TF32 products.)"""
    ctx, torch, capi = env
    M = N = K = 256
    A = (1.0 + rnd(5, M, K) * 1e-3).astype(np.float32)
    B = (1.0 + rnd(6, K, N) * 1e-3).astype(np.float32)
    C = torch.empty(M, N, device="cuda")
    default = ctx.ctx_gemm_split_mode()
    assert default == int(os.environ.get("GRADC_TC_SPLIT_MODE", "2"))
    ctx.ctx_set_gemm_split_mode(mode)
    try:
        ctx.gemm_f32(0, 0, M, N, K, 1.0, torch.from_numpy(A).cuda(), K, torch.from_numpy(B).cuda(), N, 0.0, C, N, None)
        ctx.sync()
    finally:
        ctx.ctx_set_gemm_split_mode(default)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    assert float(np.abs(C.cpu().numpy() - ref).max() / np.abs(ref).max()) < 1e-5


@pytest.mark.parametrize("opa,opb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_split_modes_agree_on_zero_mean_operands(env, opa, opb):
    """N(0,1) operands in every storage orientation (the splitter reads K-major and MN-major raw tiles differently), a shape
    that runs the CTA-pair kernel and one that runs the single-CTA kernel: both split modes within 5e-6 of fp64."""
    ctx, torch, capi = env
    default = ctx.ctx_gemm_split_mode()
    try:
        for (M, N, K) in [(512, 512, 512), (256, 192, 80)]:
            A = rnd(40, *((K, M) if opa else (M, K)))
            B = rnd(41, *((N, K) if opb else (K, N)))
            ref = (A.T if opa else A).astype(np.float64) @ (B.T if opb else B).astype(np.float64)
            for mode in (2, 1):
                ctx.ctx_set_gemm_split_mode(mode)
                C = torch.empty(M, N, device="cuda")
                ctx.gemm_f32(opa, opb, M, N, K, 1.0, torch.from_numpy(A).cuda(), A.shape[1], torch.from_numpy(B).cuda(), B.shape[1], 0.0, C, N, None)
                ctx.sync()
                assert max_abs_rel(C.cpu().numpy(), ref) < 5e-6, (mode, M, N, K)
    finally:
        ctx.ctx_set_gemm_split_mode(default)


def test_tc_gemm_head_strided_batches(env):
    """q k^T and p v on (B, T, H*D) buffers addressed through two-level batch strides, output written head-interleaved."""
    ctx, torch, capi = env
    Bn, H, T, D = 2, 3, 160, 64
    C = H * D
    q, k, v = rnd(7, Bn, T, C), rnd(8, Bn, T, C), rnd(9, Bn, T, C)
    Q, Kd, Vd = (torch.from_numpy(x).cuda() for x in (q, k, v))
    S = torch.empty(Bn * H, T, T, device="cuda")
    ctx.gemm_batched_f32(0, 1, T, T, D, 1.0, Q, C, T * C, D, Kd, C, T * C, D, 0.0, S, T, H * T * T, T * T, Bn, H)
    ctx.sync()
    qh = q.reshape(Bn, T, H, D).transpose(0, 2, 1, 3).astype(np.float64)
    kh = k.reshape(Bn, T, H, D).transpose(0, 2, 1, 3).astype(np.float64)
    vh = v.reshape(Bn, T, H, D).transpose(0, 2, 1, 3).astype(np.float64)
    ref_s = qh @ kh.transpose(0, 1, 3, 2)
    assert max_abs_rel(S.cpu().numpy().reshape(Bn, H, T, T), ref_s) < TOL
    O = torch.zeros(Bn, T, C, device="cuda")
    ctx.gemm_batched_f32(0, 0, T, D, T, 1.0, S, T, H * T * T, T * T, Vd, C, T * C, D, 0.0, O, C, T * C, D, Bn, H)
    ctx.sync()
    ref_o = (S.cpu().numpy().reshape(Bn, H, T, T).astype(np.float64) @ vh).transpose(0, 2, 1, 3).reshape(Bn, T, C)
    assert max_abs_rel(O.cpu().numpy(), ref_o) < TOL
    dV = torch.zeros(Bn, T, C, device="cuda")  # P^T . dO with A transposed
    ctx.gemm_batched_f32(1, 0, T, D, T, 1.0, S, T, H * T * T, T * T, Q, C, T * C, D, 0.0, dV, C, T * C, D, Bn, H)
    ctx.sync()
    ref_dv = (S.cpu().numpy().reshape(Bn, H, T, T).astype(np.float64).transpose(0, 1, 3, 2) @ qh).transpose(0, 2, 1, 3).reshape(Bn, T, C)
    assert max_abs_rel(dV.cpu().numpy(), ref_dv) < TOL


def test_unaligned_operands_fall_back_or_fail_loudly(env):
    ctx, torch, capi = env
    A, B = rnd(10, 64, 130), rnd(11, 130, 66)  # ld 130 / 66: not multiples of four floats
    C = torch.empty(64, 66, device="cuda")
    with pytest.raises(capi.GcbError) as e:  # engine forced to tcgen05: must refuse, not silently take another path
        ctx.gemm_f32(0, 0, 64, 66, 130, 1.0, torch.from_numpy(A).cuda(), 130, torch.from_numpy(B).cuda(), 66, 0.0, C, 66, None)
    assert e.value.status == capi.UNSUPPORTED
    ctx.ctx_set_gemm_engine(0)
    ctx.gemm_f32(0, 0, 64, 66, 130, 1.0, torch.from_numpy(A).cuda(), 130, torch.from_numpy(B).cuda(), 66, 0.0, C, 66, None)
    ctx.sync()
    assert ctx.ctx_last_gemm_engine() == 1
    assert max_abs_rel(C.cpu().numpy(), A.astype(np.float64) @ B.astype(np.float64)) < 1e-5
    ctx.ctx_set_gemm_engine(2)


@pytest.mark.parametrize("engine", [2, 1])
def test_causal_batched_gemms_skip_only_known_zeros(env, engine):
    ctx, torch, capi = env
    ctx.ctx_set_gemm_engine(engine)
    try:
        Bn, H, T, D = 2, 2, 384, 64
        C = H * D
        q, k, v = rnd(20, Bn, T, C), rnd(21, Bn, T, C), rnd(22, Bn, T, C)
        Q, Kd, Vd = (torch.from_numpy(x).cuda() for x in (q, k, v))
        heads = lambda a: a.reshape(Bn, T, H, D).transpose(0, 2, 1, 3).astype(np.float64)
        S = torch.full((Bn * H, T, T), float("nan"), device="cuda")  # poison: skipped tiles must never be read downstream
        ctx.gemm_batched_causal_f32(0, 1, T, T, D, 1.0, Q, C, T * C, D, Kd, C, T * C, D, 0.0, S, T, H * T * T, T * T, Bn, H, 1)
        ctx.sync()
        s = S.cpu().numpy().reshape(Bn, H, T, T)
        ref = heads(q) @ heads(k).transpose(0, 1, 3, 2)
        low = np.tril(np.ones((T, T), bool))
        assert float(np.abs(s[..., low] - ref[..., low]).max() / np.abs(ref).max()) < TOL
        ctx.causal_softmax_fwd_f32(S, S, 0.125, Bn * H * T, T)
        ctx.sync()
        p = S.cpu().numpy().reshape(Bn, H, T, T).astype(np.float64)
        assert np.isfinite(p).all() and np.all(np.triu(p, 1) == 0)
        O = torch.zeros(Bn, T, C, device="cuda")
        ctx.gemm_batched_causal_f32(0, 0, T, D, T, 1.0, S, T, H * T * T, T * T, Vd, C, T * C, D, 0.0, O, C, T * C, D, Bn, H, 2)
        dV = torch.zeros(Bn, T, C, device="cuda")
        ctx.gemm_batched_causal_f32(1, 0, T, D, T, 1.0, S, T, H * T * T, T * T, Q, C, T * C, D, 0.0, dV, C, T * C, D, Bn, H, 3)
        ctx.sync()
        untok = lambda a: a.transpose(0, 2, 1, 3).reshape(Bn, T, C)
        assert max_abs_rel(O.cpu().numpy(), untok(p @ heads(v))) < TOL
        assert max_abs_rel(dV.cpu().numpy(), untok(p.transpose(0, 1, 3, 2) @ heads(q))) < TOL
    finally:
        ctx.ctx_set_gemm_engine(2)


@pytest.mark.parametrize("engine", [2, 1])
@pytest.mark.parametrize("T", [384, 200])
def test_softmax_backward_in_the_dp_gemm_epilogue(env, engine, T):
    """dS = scale * P * (dO V^T - dO . O) from one GEMM call equals the unfused chain dP GEMM -> causal-softmax backward."""
    ctx, torch, capi = env
    ctx.ctx_set_gemm_engine(engine)
    try:
        Bn, H, D = 2, 3, 64
        C = H * D
        scale = 0.125
        q, k, v, do = rnd(30, Bn, T, C), rnd(31, Bn, T, C), rnd(32, Bn, T, C), rnd(33, Bn, T, C) * 1e-2
        heads = lambda a: a.reshape(Bn, T, H, D).transpose(0, 2, 1, 3).astype(np.float64)
        s = heads(q) @ heads(k).transpose(0, 1, 3, 2) * scale
        s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        o = p @ heads(v)
        dp = heads(do) @ heads(v).transpose(0, 1, 3, 2)
        ref = scale * p * (dp - (dp * p).sum(-1, keepdims=True))
        P = torch.from_numpy(p.reshape(Bn * H, T, T).astype(np.float32)).cuda()
        O = torch.from_numpy(o.transpose(0, 2, 1, 3).reshape(Bn, T, C).astype(np.float32)).cuda()
        dO, Vd = torch.from_numpy(do).cuda(), torch.from_numpy(v).cuda()
        rd = torch.empty(Bn * H * T, device="cuda")
        ctx.rowdot_batched_f32(rd, dO, C, T * C, D, O, C, T * C, D, T, D, Bn, H)
        ctx.sync()
        want_rd = (heads(do) * o).sum(-1).reshape(-1)
        assert max_abs_rel(rd.cpu().numpy(), want_rd) < 1e-6
        dS = torch.full((Bn * H, T, T), float("nan"), device="cuda")
        ctx.gemm_batched_softmax_bwd_f32(0, 1, T, D, 1.0, dO, C, T * C, D, Vd, C, T * C, D, dS, T, H * T * T, T * T, Bn, H, P, rd, scale)
        ctx.sync()
        got = dS.cpu().numpy().reshape(Bn, H, T, T)
        low = np.tril(np.ones((T, T), bool))
        assert np.isfinite(got[..., low]).all()
        assert float(np.abs(got[..., low] - ref[..., low]).max() / np.abs(ref).max()) < 2e-5
        # inside the 128-wide diagonal blocks everything above the diagonal is an explicit zero (the dQ / dK GEMMs read it)
        blk = (np.arange(T)[:, None] // 128) == (np.arange(T)[None, :] // 128)
        assert np.all(got[..., blk & ~low] == 0)
    finally:
        ctx.ctx_set_gemm_engine(2)


@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (384, 320, 512), (96, 80, 48)])
@pytest.mark.parametrize("opb", [1, 0])
def test_gelu_backward_in_the_gemm_epilogue(env, M, N, K, opb):
    """dpre = (dy W^T) * gelu'(pre) from one call (CTA-pair kernel where the shape allows, two passes otherwise) against float64."""
    ctx, torch, capi = env
    dy, pre = rnd(50, M, K) * 1e-2, rnd(51, M, N) * 1.5
    W = rnd(52, *((N, K) if opb else (K, N)))
    w = (W.T if opb else W).astype(np.float64)
    a, b = 0.7978845608, 0.044715
    x = pre.astype(np.float64)
    t = np.tanh(a * (x + b * x ** 3))
    ref = (dy.astype(np.float64) @ w) * (0.5 * (1 + t) + 0.5 * x * (1 - t * t) * a * (1 + 3 * b * x * x))
    out = torch.full((M, N), float("nan"), device="cuda")
    ctx.ctx_set_gemm_engine(0)
    try:
        ctx.gemm_gelu_bwd_f32(0, opb, M, N, K, torch.from_numpy(dy).cuda(), K, torch.from_numpy(W).cuda(), W.shape[1], torch.from_numpy(pre).cuda(), out)
        ctx.sync()
    finally:
        ctx.ctx_set_gemm_engine(2)
    assert max_abs_rel(out.cpu().numpy(), ref) < 1e-5


@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (96, 80, 48)])
def test_linear_gelu_forward_two_outputs(env, M, N, K):
    """pre = x W + b and act = gelu(pre) from one call; act must be gelu of exactly the pre that was stored."""
    ctx, torch, capi = env
    x, W, bias = rnd(60, M, K), rnd(61, K, N) * 0.1, rnd(62, N)
    pre, act = torch.full((M, N), float("nan"), device="cuda"), torch.full((M, N), float("nan"), device="cuda")
    ctx.ctx_set_gemm_engine(0)
    try:
        ctx.linear_gelu_fwd_f32(0, M, N, K, torch.from_numpy(x).cuda(), K, torch.from_numpy(W).cuda(), N, torch.from_numpy(bias).cuda(), pre, act)
        ctx.sync()
    finally:
        ctx.ctx_set_gemm_engine(2)
    ref = x.astype(np.float64) @ W.astype(np.float64) + bias
    assert max_abs_rel(pre.cpu().numpy(), ref) < 1e-5
    again = torch.empty_like(pre)
    ctx.gelu_fwd_f32(again, pre, M * N)
    ctx.sync()
    assert torch.equal(again, act)


@pytest.mark.parametrize("M,N,K,opb,with_bias", [(512, 512, 256, 0, True), (768, 256, 1024, 1, False), (96, 80, 48, 0, True), (300, 260, 64, 1, True)])
def test_linear_with_residual_epilogue(env, M, N, K, opb, with_bias):
    """out = (x op(W) + b) + r from one call: the CTA-pair kernel's residual epilogue (whole and ragged tiles) and the two-pass
    fallback for shapes it does not take, against float64; where the plain GEMM runs unsliced the result equals GEMM + add bit
    for bit (same order of additions)."""
    ctx, torch, capi = env
    x, W, bias, r = rnd(80, M, K), (rnd(81, N, K) if opb else rnd(81, K, N)) * 0.1, rnd(82, N), rnd(83, M, N) * 3
    X, Wd, Bd, R = (torch.from_numpy(a).cuda() for a in (x, W, bias, r))
    out = torch.full((M, N), float("nan"), device="cuda")
    ctx.ctx_set_gemm_engine(0)
    try:
        before = ctx.ctx_launch_count_named(b"gemm_tc_pair_residual")
        ctx.linear_residual_f32(opb, M, N, K, X, K, Wd, W.shape[1], Bd if with_bias else None, R, out)
        plain = torch.empty_like(out)
        ctx.gemm_f32(0, opb, M, N, K, 1.0, X, K, Wd, W.shape[1], 0.0, plain, N, Bd if with_bias else None)
        ctx.binary_f32(0, plain, plain, R, M * N)  # GCB_B_ADD
        ctx.sync()
        fused = ctx.ctx_launch_count_named(b"gemm_tc_pair_residual") - before
    finally:
        ctx.ctx_set_gemm_engine(2)
    ref = x.astype(np.float64) @ (W.T if opb else W).astype(np.float64) + (bias if with_bias else 0.0) + r
    assert max_abs_rel(out.cpu().numpy(), ref) < 1e-5
    if K < 1024:  # longer K loops on few tiles make the plain GEMM cut K into slices, which the residual form does not: another summation order
        assert torch.equal(out, plain)
    else:
        assert max_abs_rel(out.cpu().numpy(), plain.cpu().numpy()) < 1e-5
    assert fused == (1 if M > 128 and N > 128 and K >= 256 else 0)  # small or short-K shapes go through the fallback
    with pytest.raises(capi.GcbError) as e:
        ctx.linear_residual_f32(opb, M, N, K, X, K, Wd, W.shape[1], None, out, out)  # out aliases the residual
    assert e.value.status == capi.INVALID_ARG


def test_pair_kernel_batched_and_causal_paths(env):
    """Head dimension 256 sends every attention GEMM to the CTA-pair kernel (N = 256 or K >= 256): batched operands with
    two-level strides and all three causal variants there, against float64."""
    ctx, torch, capi = env
    Bn, H, T, D = 2, 2, 512, 256
    C = H * D
    q, k, v = rnd(70, Bn, T, C), rnd(71, Bn, T, C), rnd(72, Bn, T, C)
    Q, Kd, Vd = (torch.from_numpy(x).cuda() for x in (q, k, v))
    heads = lambda a: a.reshape(Bn, T, H, D).transpose(0, 2, 1, 3).astype(np.float64)
    untok = lambda a: a.transpose(0, 2, 1, 3).reshape(Bn, T, C)
    low = np.tril(np.ones((T, T), bool))
    S = torch.full((Bn * H, T, T), float("nan"), device="cuda")
    ctx.gemm_batched_causal_f32(0, 1, T, T, D, 1.0, Q, C, T * C, D, Kd, C, T * C, D, 0.0, S, T, H * T * T, T * T, Bn, H, 1)
    ctx.sync()
    assert ctx.ctx_last_gemm_engine() == 2
    ref = heads(q) @ heads(k).transpose(0, 1, 3, 2)
    s = S.cpu().numpy().reshape(Bn, H, T, T)
    assert float(np.abs(s[..., low] - ref[..., low]).max() / np.abs(ref).max()) < TOL
    Sf = torch.empty(Bn * H, T, T, device="cuda")
    ctx.gemm_batched_f32(0, 1, T, T, D, 1.0, Q, C, T * C, D, Kd, C, T * C, D, 0.0, Sf, T, H * T * T, T * T, Bn, H)
    ctx.sync()
    assert max_abs_rel(Sf.cpu().numpy().reshape(Bn, H, T, T), ref) < TOL
    p = np.tril(np.abs(ref) / np.abs(ref).sum(-1, keepdims=True))  # any lower-triangular matrix will do
    P = torch.from_numpy(p.reshape(Bn * H, T, T).astype(np.float32)).cuda()
    p = P.cpu().numpy().reshape(Bn, H, T, T).astype(np.float64)
    O = torch.zeros(Bn, T, C, device="cuda")
    ctx.gemm_batched_causal_f32(0, 0, T, D, T, 1.0, P, T, H * T * T, T * T, Vd, C, T * C, D, 0.0, O, C, T * C, D, Bn, H, 2)
    dV = torch.zeros(Bn, T, C, device="cuda")
    ctx.gemm_batched_causal_f32(1, 0, T, D, T, 1.0, P, T, H * T * T, T * T, Q, C, T * C, D, 0.0, dV, C, T * C, D, Bn, H, 3)
    ctx.sync()
    assert max_abs_rel(O.cpu().numpy(), untok(p @ heads(v))) < TOL
    assert max_abs_rel(dV.cpu().numpy(), untok(p.transpose(0, 1, 3, 2) @ heads(q))) < TOL


def test_fused_entry_points_accept_empty_problems_and_reject_bad_arguments(env):
    """Zero-sized calls are no-ops; aliasing and missing operands are refused with GCB_INVALID_ARG before any launch."""
    ctx, torch, capi = env
    z = torch.zeros(16, device="cuda")
    ctx.rowdot_batched_f32(z, z, 4, 0, 0, z, 4, 0, 0, 0, 4, 1, 1)           # no rows
    ctx.rowdot_batched_f32(z, z, 4, 0, 0, z, 4, 0, 0, 4, 4, 0, 3)           # no batch items
    ctx.gemm_batched_softmax_bwd_f32(0, 1, 0, 8, 1.0, z, 8, 0, 0, z, 8, 0, 0, z, 4, 0, 0, 1, 1, z[4:], z, 1.0)  # M = 0
    ctx.gemm_gelu_bwd_f32(0, 0, 0, 4, 4, z, 4, z, 4, z, z[4:])              # M = 0 (pre / dpre only have to differ)
    ctx.sync()
    with pytest.raises(capi.GcbError) as e:
        ctx.gemm_gelu_bwd_f32(0, 0, 4, 4, 4, z, 4, z, 4, z, z)              # dpre aliases pre
    assert e.value.status == capi.INVALID_ARG
    with pytest.raises(capi.GcbError) as e:
        ctx.linear_gelu_fwd_f32(0, 4, 4, 4, z, 4, z, 4, None, z, z)         # act aliases pre
    assert e.value.status == capi.INVALID_ARG
    with pytest.raises(capi.GcbError) as e:
        ctx.gemm_batched_softmax_bwd_f32(0, 1, 4, 4, 1.0, z, 4, 0, 0, z, 4, 0, 0, z, 4, 0, 0, 1, 1, None, z, 1.0)  # no probabilities
    assert e.value.status == capi.INVALID_ARG
    with pytest.raises(capi.GcbError) as e:
        ctx.ctx_set_gemm_split_mode(7)
    assert e.value.status == capi.INVALID_ARG


def test_causal_attention_gemms_over_several_scheduling_groups(env):
    """The six attention GEMMs of a training step on 80 heads of 1024 x 64: the 64-wide causal kernels deal their tiles in
    groups of 2 x 148 / 8 = 37 heads (snake order inside a group), so 80 heads make two full groups and a ragged last one of
    6, with the persistent loop rounded up past the last item.  Heads from the first group, a group boundary and the tail are
    checked against float64 (full tensors would take minutes on the host)."""
    ctx, torch, capi = env
    Bn, H, T, D = 5, 16, 1024, 64
    C = H * D
    scale = 0.125
    q, k, v, do = rnd(80, Bn, T, C), rnd(81, Bn, T, C), rnd(82, Bn, T, C), rnd(83, Bn, T, C) * 1e-2
    Q, Kd, Vd, dO = (torch.from_numpy(x).cuda() for x in (q, k, v, do))
    head = lambda a, i: a[i // H, :, (i % H) * D:(i % H + 1) * D].astype(np.float64)   # (T, D) of batch item i
    low = np.tril(np.ones((T, T), bool))
    blk = (np.arange(T)[:, None] // 128) == (np.arange(T)[None, :] // 128)
    sample = [0, 1, 36, 37, 38, 73, 74, 75, 79]
    # forward: scores (causal 1) -> band softmax -> P V (causal 2), as SDPANode::realize issues them
    S = torch.full((Bn * H, T, T), float("nan"), device="cuda")
    ctx.gemm_batched_causal_f32(0, 1, T, T, D, 1.0, Q, C, T * C, D, Kd, C, T * C, D, 0.0, S, T, H * T * T, T * T, Bn, H, 1)
    ctx.sync()
    assert ctx.ctx_last_gemm_engine() == 2
    for i in sample:
        ref = head(q, i) @ head(k, i).T
        got = S[i].cpu().numpy()
        assert float(np.abs(got[low] - ref[low]).max() / np.abs(ref).max()) < TOL, i
    ctx.causal_softmax_fwd_band_f32(S, S, scale, Bn * H * T, T, 128)
    Oo = torch.full((Bn, T, C), float("nan"), device="cuda")
    ctx.gemm_batched_causal_f32(0, 0, T, D, T, 1.0, S, T, H * T * T, T * T, Vd, C, T * C, D, 0.0, Oo, C, T * C, D, Bn, H, 2)
    ctx.sync()
    o_host = Oo.cpu().numpy()
    assert np.isfinite(o_host).all()
    probs = {}
    for i in sample:
        s = np.where(low, head(q, i) @ head(k, i).T * scale, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        probs[i] = p
        got_p = S[i].cpu().numpy()
        assert float(np.abs(np.where(low, got_p, 0) - p).max()) < 1e-5, i
        assert max_abs_rel(o_host[i // H, :, (i % H) * D:(i % H + 1) * D], p @ head(v, i)) < TOL, i
    # backward: dV = P^T dO (causal 3), dS from the dP GEMM with the softmax backward in its epilogue, dQ = dS K (causal 2), dK = dS^T Q (causal 3)
    dV, dQ, dK = (torch.full((Bn, T, C), float("nan"), device="cuda") for _ in range(3))
    ctx.gemm_batched_causal_f32(1, 0, T, D, T, 1.0, S, T, H * T * T, T * T, dO, C, T * C, D, 0.0, dV, C, T * C, D, Bn, H, 3)
    rd = torch.empty(Bn * H * T, device="cuda")
    ctx.rowdot_batched_f32(rd, dO, C, T * C, D, Oo, C, T * C, D, T, D, Bn, H)
    dS = torch.full((Bn * H, T, T), float("nan"), device="cuda")
    ctx.gemm_batched_softmax_bwd_f32(0, 1, T, D, 1.0, dO, C, T * C, D, Vd, C, T * C, D, dS, T, H * T * T, T * T, Bn, H, S, rd, scale)
    ctx.gemm_batched_causal_f32(0, 0, T, D, T, 1.0, dS, T, H * T * T, T * T, Kd, C, T * C, D, 0.0, dQ, C, T * C, D, Bn, H, 2)
    ctx.gemm_batched_causal_f32(1, 0, T, D, T, 1.0, dS, T, H * T * T, T * T, Q, C, T * C, D, 0.0, dK, C, T * C, D, Bn, H, 3)
    ctx.sync()
    dv_h, dq_h, dk_h = dV.cpu().numpy(), dQ.cpu().numpy(), dK.cpu().numpy()
    assert np.isfinite(dv_h).all() and np.isfinite(dq_h).all() and np.isfinite(dk_h).all()
    for i in sample:
        p = probs[i]
        dp = head(do, i) @ head(v, i).T
        ds = scale * p * (dp - (dp * p).sum(-1, keepdims=True))
        got = dS[i].cpu().numpy()
        assert float(np.abs(got[low] - ds[low]).max() / np.abs(ds).max()) < TOL, i
        assert np.all(got[blk & ~low] == 0), i
        sl = (i // H, slice(None), slice((i % H) * D, (i % H + 1) * D))
        assert max_abs_rel(dv_h[sl], p.T @ head(do, i)) < TOL, i
        assert max_abs_rel(dq_h[sl], ds @ head(k, i)) < TOL, i
        assert max_abs_rel(dk_h[sl], ds.T @ head(q, i)) < TOL, i


def test_fused_epilogues_take_the_scalar_path_for_side_arrays_off_a_16_byte_boundary(env):
    """The epilogues read the probabilities / pre-activations and write the activations with 16-byte vector accesses only when
    those arrays sit on 16-byte boundaries like C; a side array at a 4-byte offset must give the same result through the
    scalar path (not a misaligned-address fault)."""
    ctx, torch, capi = env
    Bn, H, T, D = 1, 2, 256, 64
    C = H * D
    scale = 0.125
    v, do = rnd(90, Bn, T, C), rnd(91, Bn, T, C) * 1e-2
    p = np.tril(np.abs(rnd(92, Bn * H, T, T)))
    p = (p / p.sum(-1, keepdims=True)).astype(np.float32)
    rdot = rnd(93, Bn * H * T) * 1e-2
    buf = torch.zeros(p.size + 4, device="cuda")
    P_off = buf[1:1 + p.size]
    P_off.copy_(torch.from_numpy(p.reshape(-1)))
    assert P_off.data_ptr() % 16 == 4
    dO, Vd, RD = torch.from_numpy(do).cuda(), torch.from_numpy(v).cuda(), torch.from_numpy(rdot).cuda()
    dS = torch.full((Bn * H, T, T), float("nan"), device="cuda")
    ctx.gemm_batched_softmax_bwd_f32(0, 1, T, D, 1.0, dO, C, T * C, D, Vd, C, T * C, D, dS, T, H * T * T, T * T, Bn, H, P_off, RD, scale)
    ctx.sync()
    heads = lambda a: a.reshape(Bn, T, H, D).transpose(0, 2, 1, 3).astype(np.float64).reshape(Bn * H, T, D)
    dp = heads(do) @ heads(v).transpose(0, 2, 1)
    ref = scale * p.astype(np.float64) * (dp - rdot.astype(np.float64).reshape(Bn * H, T, 1))
    low = np.tril(np.ones((T, T), bool))
    got = dS.cpu().numpy()
    assert float(np.abs(got[:, low] - ref[:, low]).max() / np.abs(ref).max()) < TOL
    # GELU epilogues of the CTA-pair kernel with pre / act at a 4-byte offset
    M, N, K = 512, 512, 256
    x, W, bias = rnd(94, M, K), rnd(95, K, N) * 0.1, rnd(96, N)
    pre = torch.empty(M, N, device="cuda")
    abuf = torch.zeros(M * N + 4, device="cuda")
    act_off = abuf[1:1 + M * N]
    ctx.linear_gelu_fwd_f32(0, M, N, K, torch.from_numpy(x).cuda(), K, torch.from_numpy(W).cuda(), N, torch.from_numpy(bias).cuda(), pre, act_off)
    again = torch.empty_like(pre)
    ctx.gelu_fwd_f32(again, pre, M * N)
    ctx.sync()
    assert max_abs_rel(pre.cpu().numpy(), x.astype(np.float64) @ W.astype(np.float64) + bias) < 1e-5
    assert torch.equal(again.reshape(-1), act_off)
    pbuf = torch.zeros(M * N + 4, device="cuda")
    pre_off = pbuf[1:1 + M * N]
    pre_off.copy_(pre.reshape(-1))
    dy, W2 = rnd(97, M, K) * 1e-2, rnd(98, N, K)
    out_a, out_b = torch.empty(M, N, device="cuda"), torch.empty(M, N, device="cuda")
    ctx.gemm_gelu_bwd_f32(0, 1, M, N, K, torch.from_numpy(dy).cuda(), K, torch.from_numpy(W2).cuda(), K, pre, out_a)
    ctx.gemm_gelu_bwd_f32(0, 1, M, N, K, torch.from_numpy(dy).cuda(), K, torch.from_numpy(W2).cuda(), K, pre_off, out_b)
    ctx.sync()
    assert ctx.ctx_launch_count_named(b"gemm_tc_pair_gelu_bwd") >= 2
    assert torch.equal(out_a, out_b)


@pytest.mark.parametrize("Kin,Nout,Mtok,family", [(1024, 1024, 8192, "gemm_tc_pair"), (512, 768, 4096, "gemm_tc_pair"), (256, 1024, 300, "gemm_tc_pair"), (96, 80, 200, None), (1024, 100, 4096, None)])
def test_weight_gradient_with_bias_gradient_from_one_pass(env, Kin, Nout, Mtok, family):
    """dW = x^T dy and db = column sums of dy from one call, against float64: shapes that run the CTA-pair kernel with and
    without K slices (the B-splitter warps gather the sums), and shapes that fall back to the product plus a row reduction.
    Overwrite and accumulate forms; the result is run-to-run identical."""
    ctx, torch, capi = env
    x, dy = rnd(100, Mtok, Kin), rnd(101, Mtok, Nout) * 1e-2 + 3e-3
    dW0, db0 = rnd(102, Kin, Nout) * 1e-2, rnd(103, Nout) * 1e-2
    X, DY = torch.from_numpy(x).cuda(), torch.from_numpy(dy).cuda()
    ref_w = x.astype(np.float64).T @ dy.astype(np.float64)
    ref_b = dy.astype(np.float64).sum(0)
    ctx.ctx_set_gemm_engine(0)
    try:
        before = ctx.ctx_launch_count_named(b"gemm_tc_pair")
        dW, db = torch.full((Kin, Nout), float("nan"), device="cuda"), torch.full((Nout,), float("nan"), device="cuda")
        ctx.gemm_colsum_f32(1, Kin, Nout, Mtok, 1.0, X, Kin, DY, 0.0, dW, Nout, db, 0)
        ctx.sync()
        if family:
            assert ctx.ctx_launch_count_named(b"gemm_tc_pair") == before + 1
        assert max_abs_rel(dW.cpu().numpy(), ref_w) < TOL and max_abs_rel(db.cpu().numpy(), ref_b) < 1e-5
        first = (dW.clone(), db.clone())
        dW2, db2 = torch.from_numpy(dW0).cuda(), torch.from_numpy(db0).cuda()
        ctx.gemm_colsum_f32(1, Kin, Nout, Mtok, 1.0, X, Kin, DY, 1.0, dW2, Nout, db2, 1)
        ctx.sync()
        assert max_abs_rel(dW2.cpu().numpy(), ref_w + dW0) < TOL and max_abs_rel(db2.cpu().numpy(), ref_b + db0) < 1e-5
        dW3, db3 = torch.empty_like(dW), torch.empty_like(db)
        ctx.gemm_colsum_f32(1, Kin, Nout, Mtok, 1.0, X, Kin, DY, 0.0, dW3, Nout, db3, 0)
        ctx.sync()
        assert torch.equal(dW3, first[0]) and torch.equal(db3, first[1])
    finally:
        ctx.ctx_set_gemm_engine(2)


def test_bias_gradient_rides_on_the_pair_kernel_for_the_step_shapes(env):
    """At a linear layer's backward shape the fused call launches the pair GEMM (+ its K-slice reduction) and no row-reduction kernel."""
    ctx, torch, capi = env
    Kin, Nout, Mtok = 1024, 1024, 8192
    X, DY = torch.from_numpy(rnd(110, Mtok, Kin)).cuda(), torch.from_numpy(rnd(111, Mtok, Nout)).cuda()
    dW, db = torch.empty(Kin, Nout, device="cuda"), torch.empty(Nout, device="cuda")
    pair0, red0 = ctx.ctx_launch_count_named(b"gemm_tc_pair"), ctx.ctx_launch_count_named(b"reduce_rows")
    ctx.gemm_colsum_f32(1, Kin, Nout, Mtok, 1.0, X, Kin, DY, 0.0, dW, Nout, db, 0)
    ctx.sync()
    assert ctx.ctx_launch_count_named(b"gemm_tc_pair") == pair0 + 1
    assert ctx.ctx_launch_count_named(b"reduce_rows") == red0
    assert max_abs_rel(db.cpu().numpy(), DY.double().sum(0).cpu().numpy()) < 1e-5


@pytest.mark.parametrize("rows,cols,M", [(1024, 768, 4096), (1000, 520, 700), (256, 1024, 384)])
def test_registered_weights_use_presplit_companions_with_identical_results(env, rows, cols, M):
    """A weight registered with gcb_weight_twins_register keeps its BF16 companions pre-split in global memory; the CTA-pair
    kernel then fetches them by TMA instead of deriving them in every CTA.  Same values, so the product is bit-identical with
    and without registration, in both roles of the weight (y = x W and dx = dy W^T), with ragged edges; a write into the
    weight through the library makes the next GEMM recompute the companions."""
    ctx, torch, capi = env
    w = rnd(120, rows, cols) * 0.05
    x, dy = rnd(121, M, rows), rnd(122, M, cols) * 1e-2
    W_plain, W_reg = torch.from_numpy(w).cuda(), torch.from_numpy(w).cuda()
    X, DY = torch.from_numpy(x).cuda(), torch.from_numpy(dy).cuda()

    def products(W):
        y, dx = torch.full((M, cols), float("nan"), device="cuda"), torch.full((M, rows), float("nan"), device="cuda")
        ctx.gemm_f32(0, 0, M, cols, rows, 1.0, X, rows, W, cols, 0.0, y, cols, None)
        ctx.gemm_f32(0, 1, M, rows, cols, 1.0, DY, cols, W, cols, 0.0, dx, rows, None)
        ctx.sync()
        return y, dx

    y0, dx0 = products(W_plain)
    assert max_abs_rel(y0.cpu().numpy(), x.astype(np.float64) @ w.astype(np.float64)) < TOL
    assert max_abs_rel(dx0.cpu().numpy(), dy.astype(np.float64) @ w.astype(np.float64).T) < TOL
    n0 = ctx.weight_twins_count()
    ctx.weight_twins_register(W_reg, rows, cols)
    try:
        assert ctx.weight_twins_count() == n0 + 1
        pre0 = ctx.ctx_launch_count_named(b"presplit_weight")
        y1, dx1 = products(W_reg)
        assert ctx.ctx_launch_count_named(b"presplit_weight") == pre0 + 1  # one launch covers every registered weight, both orientations
        assert torch.equal(y1, y0) and torch.equal(dx1, dx0)
        y2, dx2 = products(W_reg)
        assert ctx.ctx_launch_count_named(b"presplit_weight") == pre0 + 1  # nothing was written: no recomputation
        assert torch.equal(y2, y0)
        # the weight changes through the library (as an optimizer step or a checkpoint load would change it)
        w2 = (w * 1.5 + 0.01).astype(np.float32)
        ctx.copy_h2d(W_reg, w2, w2.nbytes)
        ctx.copy_h2d(W_plain, w2, w2.nbytes)
        y3, dx3 = products(W_reg)
        y4, dx4 = products(W_plain)
        assert ctx.ctx_launch_count_named(b"presplit_weight") == pre0 + 2
        assert torch.equal(y3, y4) and torch.equal(dx3, dx4)
        assert max_abs_rel(y3.cpu().numpy(), x.astype(np.float64) @ w2.astype(np.float64)) < TOL
    finally:
        ctx.weight_twins_drop(W_reg, w.nbytes)
    assert ctx.weight_twins_count() == n0
