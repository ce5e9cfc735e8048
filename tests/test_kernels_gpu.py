"""Parity of every CUDA entry point (called through the C ABI) with the numpy oracle and the reference-made
golden fixtures.  Tolerances: integer/index results bit-exact; fp32 results max-abs-rel <= 1e-4 per tensor
(the bar the training path is held to), usually far tighter."""
import numpy as np
import pytest

from oracle import numpy_oracle as O
from oracle import synth
from tests.helpers import load_golden, max_abs_rel, split_prefix

pytestmark = pytest.mark.gpu
TOL = 1e-4


@pytest.fixture(scope="module")
def env():
    import torch

    from gradcraft_b200 import capi

    ctx = capi.Context(0)
    yield ctx, torch, capi
    ctx.sync()
    ctx.close()


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(ctx, t):
    ctx.sync()
    return t.cpu().numpy()


@pytest.fixture(scope="module")
def ops():
    g = load_golden("ops")
    return split_prefix(g, "in."), split_prefix(g, "out.")


def rnd(seed, *shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape, dtype=np.float32) * scale).astype(np.float32)


# ---- elementwise --------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 3, 1024, 4099, 1 << 20])
def test_unary_binary(env, n):
    ctx, torch, capi = env
    a, b = rnd(1, n), rnd(2, n) + 3.0
    da, db, out = dev(torch, a), dev(torch, b), torch.empty(n, device="cuda")
    for name, ref in (("ADD", a + b), ("SUB", a - b), ("MUL", a * b), ("DIV", a / b), ("ISUB", b - a), ("IDIV", b / a)):
        ctx.binary_f32(capi.B[name], out, da, db, n)
        assert max_abs_rel(host(ctx, out), ref) < 1e-6, name
    ctx.binary_f32(capi.B["BGELU"], out, da, db, n)
    assert max_abs_rel(host(ctx, out), O.gelu_bwd(a, b)) < TOL
    for name, ref in (("IDENTITY", a), ("NEG", -a), ("SQUARE", a * a), ("GELU", O.gelu_fwd(a)), ("SILU", a / (1 + np.exp(-a))), ("RELU", np.maximum(a, 0))):
        ctx.unary_f32(capi.U[name], out, da, n)
        assert max_abs_rel(host(ctx, out), ref) < 1e-5, name
    ctx.binary_scalar_f32(capi.B["DIV"], out, da, 16.0, n)
    assert max_abs_rel(host(ctx, out), a / 16.0) < 1e-6
    # in place and on a misaligned view
    if n > 8:
        v = da[1:]
        ctx.binary_scalar_f32(capi.B["MUL"], v, v, 2.0, n - 1)
        assert max_abs_rel(host(ctx, da)[1:], a[1:] * 2) < 1e-6


def test_rowvec_strided_reduce(env):
    ctx, torch, capi = env
    a, v = rnd(3, 37, 20), rnd(4, 20)
    out = torch.empty(37, 20, device="cuda")
    ctx.binary_rowvec_f32(capi.B["ADD"], out, dev(torch, a), dev(torch, v), 37, 20)
    assert np.allclose(host(ctx, out), a + v, atol=1e-6)
    a2, v2 = rnd(5, 9, 7), rnd(6, 7)
    out2 = torch.empty(9, 7, device="cuda")
    ctx.binary_rowvec_f32(capi.B["MUL"], out2, dev(torch, a2), dev(torch, v2), 9, 7)
    assert np.allclose(host(ctx, out2), a2 * v2, atol=1e-6)
    # permute copy (B,T,H,D) -> (B,H,T,D) through strides
    x = rnd(7, 2, 5, 3, 4)
    dx, y = dev(torch, x), torch.empty(2, 3, 5, 4, device="cuda")
    shape = np.array([2, 3, 5, 4], dtype=np.int64)
    so = np.array([60, 20, 4, 1], dtype=np.int64)
    si = np.array([60, 4, 12, 1], dtype=np.int64)
    ctx.copy_strided_f32(4, shape, y, so, dx, si, 0)
    assert np.array_equal(host(ctx, y), x.transpose(0, 2, 1, 3))
    ctx.copy_strided_f32(4, shape, y, so, dx, si, 1)
    assert np.allclose(host(ctx, y), 2 * x.transpose(0, 2, 1, 3))
    # broadcast add with stride 0
    b = rnd(8, 5, 4)
    z = torch.empty(2, 3, 5, 4, device="cuda")
    sb = np.array([0, 0, 4, 1], dtype=np.int64)
    ctx.binary_strided_f32(capi.B["ADD"], 4, shape, z, so, dx, si, dev(torch, b), sb)
    assert np.allclose(host(ctx, z), x.transpose(0, 2, 1, 3) + b, atol=1e-6)
    for rows, cols in ((1, 5), (300, 20), (4096, 1024), (1000, 33)):
        m = rnd(9, rows, cols)
        r = torch.full((cols,), 1.0, device="cuda")
        ctx.reduce_rows_f32(r, dev(torch, m), rows, cols, 0)
        assert max_abs_rel(host(ctx, r), m.sum(0, dtype=np.float64)) < 1e-5
        ctx.reduce_rows_f32(r, dev(torch, m), rows, cols, 1)
        assert max_abs_rel(host(ctx, r), 2 * m.sum(0, dtype=np.float64)) < 1e-5
    for n in (1, 1000, 1 << 20):
        g = rnd(10, n)
        s = torch.zeros(1, device="cuda")
        ctx.sum_squares_f32(s, dev(torch, g), n, 0)
        assert abs(float(host(ctx, s)[0]) - float((g.astype(np.float64) ** 2).sum())) / float((g.astype(np.float64) ** 2).sum()) < 1e-6


def test_fill_and_copies(env):
    ctx, torch, capi = env
    t = torch.empty(1001, device="cuda")
    ctx.fill_f32(t, 2.5, 1001)
    assert np.all(host(ctx, t) == 2.5)
    ctx.fill_f32(t[1:], 0.0, 1000)
    assert host(ctx, t)[0] == 2.5 and np.all(host(ctx, t)[1:] == 0)
    ctx.set_scalar_f32(t, 3e-4)
    assert host(ctx, t)[0] == np.float32(3e-4)
    ar = torch.empty(64, dtype=torch.int64, device="cuda")
    ctx.fill_arange_i64(ar, 0, 1, 64)
    assert np.array_equal(host(ctx, ar), np.arange(64))
    src = rnd(11, 257)
    ctx.copy_h2d(t, src, 257 * 4)
    back = np.empty(257, np.float32)
    ctx.copy_d2h(back, t, 257 * 4)
    assert np.array_equal(back, src)


# ---- golden fixtures (reference outputs) ------------------------------------------------------------
def test_layernorm_golden(env, ops):
    ctx, torch, capi = env
    i, o = ops
    x = i["ln.x"].reshape(-1, 50)
    rows, cols = x.shape
    y, mu, rs = torch.empty(rows, cols, device="cuda"), torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    dx, dg, db = torch.empty(rows, cols, device="cuda"), torch.empty(cols, device="cuda"), torch.empty(cols, device="cuda")
    X, G, Bt, DY = dev(torch, x), dev(torch, i["ln.gamma"]), dev(torch, i["ln.beta"]), dev(torch, i["ln.dy"].reshape(-1, 50))
    ctx.layernorm_fwd_f32(y, mu, rs, X, G, Bt, rows, cols, float(i["ln.eps"][0]))
    ctx.layernorm_bwd_f32(dx, dg, db, DY, X, G, mu, rs, rows, cols, 0, 0)
    assert max_abs_rel(host(ctx, y), o["ln.y"].reshape(rows, cols)) < TOL
    assert max_abs_rel(host(ctx, dx), o["ln.dx"].reshape(rows, cols)) < TOL
    assert max_abs_rel(host(ctx, dg), o["ln.dgamma"]) < TOL
    assert max_abs_rel(host(ctx, db), o["ln.dbeta"]) < TOL


def test_rmsnorm_golden(env, ops):
    ctx, torch, capi = env
    i, o = ops
    x = i["rms.x"].reshape(-1, 50)
    rows, cols = x.shape
    y, inv = torch.empty(rows, cols, device="cuda"), torch.empty(rows, device="cuda")
    dx, dg = torch.empty(rows, cols, device="cuda"), torch.empty(cols, device="cuda")
    X, G, DY = dev(torch, x), dev(torch, i["rms.gamma"]), dev(torch, i["rms.dy"].reshape(-1, 50))
    ctx.rmsnorm_fwd_f32(y, inv, X, G, rows, cols, float(i["rms.eps"][0]))
    ctx.rmsnorm_bwd_f32(dx, dg, DY, X, G, inv, rows, cols, 0, 0)
    assert max_abs_rel(host(ctx, y), o["rms.y"].reshape(rows, cols)) < TOL
    assert max_abs_rel(host(ctx, dx), o["rms.dx"].reshape(rows, cols)) < TOL
    assert max_abs_rel(host(ctx, dg), o["rms.dgamma"]) < TOL


def test_activations_golden(env, ops):
    ctx, torch, capi = env
    i, o = ops
    n = i["gelu.x"].size
    X, DY, out = dev(torch, i["gelu.x"]), dev(torch, i["gelu.dy"]), torch.empty(n, device="cuda")
    ctx.gelu_fwd_f32(out, X, n)
    assert max_abs_rel(host(ctx, out).reshape(i["gelu.x"].shape), o["gelu.y"]) < TOL
    ctx.gelu_bwd_f32(out, DY, X, n, 0)
    assert max_abs_rel(host(ctx, out).reshape(i["gelu.x"].shape), o["gelu.dx"]) < TOL
    ctx.gelu_bwd_f32(out, DY, X, n, 1)
    assert max_abs_rel(host(ctx, out).reshape(i["gelu.x"].shape), 2 * o["gelu.dx"]) < TOL
    A, Bv, G = dev(torch, i["swiglu.a"]), dev(torch, i["swiglu.b"]), dev(torch, i["swiglu.dy"])
    da, db = torch.empty(n, device="cuda"), torch.empty(n, device="cuda")
    ctx.swiglu_fwd_f32(out, A, Bv, n)
    assert max_abs_rel(host(ctx, out).reshape(o["swiglu.y"].shape), o["swiglu.y"]) < TOL
    ctx.swiglu_bwd_f32(da, db, G, A, Bv, n, 0, 0)
    assert max_abs_rel(host(ctx, da).reshape(o["swiglu.da"].shape), o["swiglu.da"]) < TOL
    assert max_abs_rel(host(ctx, db).reshape(o["swiglu.db"].shape), o["swiglu.db"]) < TOL
    ctx.swiglu_bwd_f32(da, db, G, A, Bv, n, 1, 1)
    assert max_abs_rel(host(ctx, da).reshape(o["swiglu.da"].shape), 2 * o["swiglu.da"]) < TOL
    assert max_abs_rel(host(ctx, db).reshape(o["swiglu.db"].shape), 2 * o["swiglu.db"]) < TOL


def test_causal_softmax_golden(env, ops):
    ctx, torch, capi = env
    i, o = ops
    s = i["csm.scores"]
    T = s.shape[-1]
    rows = s.size // T
    P, dS = torch.empty(rows, T, device="cuda"), torch.empty(rows, T, device="cuda")
    ctx.causal_softmax_fwd_f32(P, dev(torch, s), float(i["csm.scale"][0]), rows, T)
    p = host(ctx, P).reshape(s.shape)
    assert max_abs_rel(p, o["csm.probs"]) < TOL
    assert np.all(np.triu(p, 1) == 0)
    ctx.causal_softmax_bwd_f32(dS, dev(torch, i["csm.dy"]), P, float(i["csm.scale"][0]), rows, T, 0)
    assert max_abs_rel(host(ctx, dS).reshape(s.shape), o["csm.dscores"]) < TOL


def test_softmax_ce_golden(env, ops):
    ctx, torch, capi = env
    i, o = ops
    z = i["ce.logits"]
    rows, V = z.shape
    t64 = i["ce.targets"].astype(np.int64)
    for idx_type, t in ((capi.IDX_I64, t64), (capi.IDX_I32, t64.astype(np.int32))):
        Z, Tg = dev(torch, z), dev(torch, t)
        loss, P, dZ = torch.zeros(1, device="cuda"), torch.empty(rows, V, device="cuda"), torch.empty(rows, V, device="cuda")
        ctx.softmax_ce_fwd_f32(loss, P, Z, Tg, idx_type, rows, V, float(i["ce.eps"][0]))
        assert abs(float(host(ctx, loss)[0]) - float(o["ce.loss"])) / float(o["ce.loss"]) < 1e-5
        ctx.softmax_ce_bwd_f32(dZ, P, Tg, idx_type, float(i["ce.upstream"][0]), rows, V, 0)
        assert max_abs_rel(host(ctx, dZ), o["ce.dlogits"]) < TOL
        # in place over the logits / probabilities, as the training path runs it
        ctx.softmax_ce_fwd_f32(loss, Z, Z, Tg, idx_type, rows, V, float(i["ce.eps"][0]))
        ctx.softmax_ce_bwd_f32(Z, Z, Tg, idx_type, float(i["ce.upstream"][0]), rows, V, 0)
        assert max_abs_rel(host(ctx, Z), o["ce.dlogits"]) < TOL


def test_embedding_golden_and_plan(env, ops):
    ctx, torch, capi = env
    i, o = ops
    table, idx, dy = i["emb.table"], i["emb.idx"].astype(np.int64), i["emb.dy"]
    V, W = table.shape
    n = idx.size
    out = torch.empty(n, W, device="cuda")
    ctx.embed_f32(out, dev(torch, idx), capi.IDX_I64, dev(torch, table), n, W, V)
    assert np.array_equal(host(ctx, out).reshape(o["emb.y"].shape), o["emb.y"])
    d = torch.zeros(V, W, device="cuda")
    ctx.scatter_add_f32(d, dev(torch, idx), capi.IDX_I64, dev(torch, dy), n, W, V)
    assert max_abs_rel(host(ctx, d), o["emb.dtable"]) < TOL
    order, counts, offsets = torch.empty(n, dtype=torch.int32, device="cuda"), torch.empty(V, dtype=torch.int32, device="cuda"), torch.empty(V + 1, dtype=torch.int32, device="cuda")
    ctx.scatter_plan_i32(order, counts, offsets, dev(torch, idx.astype(np.int32)), capi.IDX_I32, n, V)
    ro, rc, rf = O.scatter_plan(idx, V)
    assert np.array_equal(host(ctx, order), ro) and np.array_equal(host(ctx, counts), rc) and np.array_equal(host(ctx, offsets), rf)


def test_adamw_golden(env, ops):
    ctx, torch, capi = env
    i, o = ops
    lr, b1, b2, wd, eps, steps, clip, nd = [float(x) for x in i["adamw.hyper"]]
    w = dev(torch, i["adamw.w"])
    n = w.numel()
    m, v, sq = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(1, device="cuda")
    b1p = b2p = np.float32(1.0)
    for s in range(int(steps)):
        g = dev(torch, i["adamw.g%d" % s])
        ctx.sum_squares_f32(sq, g, n, 0)
        norm = np.float32(np.sqrt(host(ctx, sq)[0]))
        assert abs(float(norm) - float(o["adamw.norm%d" % s])) / float(norm) < 1e-6
        scale = float(np.float32(clip) / (norm + np.float32(1e-6))) if norm > clip else 1.0
        b1p, b2p = np.float32(b1p * np.float32(b1)), np.float32(b2p * np.float32(b2))
        ctx.adamw_step_f32(w, m, v, g, n, lr, b1, b2, float(b1p), float(b2p), wd, eps, int(nd), scale)
    assert max_abs_rel(host(ctx, w), o["adamw.w_out"]) < 1e-6
    assert max_abs_rel(host(ctx, m).reshape(o["adamw.m_out"].shape), o["adamw.m_out"]) < 1e-5
    assert max_abs_rel(host(ctx, v).reshape(o["adamw.v_out"].shape), o["adamw.v_out"]) < 1e-5


def test_linear_attention_golden(env, ops):
    """Linear = GEMM with bias epilogue; backward = NT and TN GEMMs + row reduction; attention = strided batched GEMMs
    on (B,T,H,D)-style views + causal softmax."""
    ctx, torch, capi = env
    i, o = ops
    x, W, b, dy = i["lin.x"].reshape(-1, 24), i["lin.W"], i["lin.b"], i["lin.dy"].reshape(-1, 20)
    M, K = x.shape
    N = W.shape[1]
    X, Wd, Bd, DY = dev(torch, x), dev(torch, W), dev(torch, b), dev(torch, dy)
    y, dx, dW, dbias = torch.empty(M, N, device="cuda"), torch.empty(M, K, device="cuda"), torch.empty(K, N, device="cuda"), torch.empty(N, device="cuda")
    ctx.gemm_f32(capi.OP_N, capi.OP_N, M, N, K, 1.0, X, K, Wd, N, 0.0, y, N, Bd)
    ctx.gemm_f32(capi.OP_N, capi.OP_T, M, K, N, 1.0, DY, N, Wd, N, 0.0, dx, K, None)
    ctx.gemm_f32(capi.OP_T, capi.OP_N, K, N, M, 1.0, X, K, DY, N, 0.0, dW, N, None)
    ctx.reduce_rows_f32(dbias, DY, M, N, 0)
    assert max_abs_rel(host(ctx, y), o["lin.y"].reshape(M, N)) < TOL
    assert max_abs_rel(host(ctx, dx), o["lin.dx"].reshape(M, K)) < TOL
    assert max_abs_rel(host(ctx, dW), o["lin.dW"]) < TOL
    assert max_abs_rel(host(ctx, dbias), o["lin.db"]) < TOL
    # beta = 1 accumulates (gradient accumulation over micro-batches)
    ctx.gemm_f32(capi.OP_T, capi.OP_N, K, N, M, 1.0, X, K, DY, N, 1.0, dW, N, None)
    assert max_abs_rel(host(ctx, dW), 2 * o["lin.dW"]) < TOL

    q, k, v, do = i["attn.q"], i["attn.k"], i["attn.v"], i["attn.dy"]
    Bn, H, T, D = q.shape
    scale = 1.0 / np.sqrt(D)
    # store q,k,v as (B,T,H*D) like the projections produce them; heads are addressed through batch strides
    tok = lambda a: np.ascontiguousarray(a.transpose(0, 2, 1, 3).reshape(Bn, T, H * D))
    Q, Kd, Vd, DO = dev(torch, tok(q)), dev(torch, tok(k)), dev(torch, tok(v)), dev(torch, tok(do))
    C = H * D
    S = torch.empty(Bn * H, T, T, device="cuda")
    Oo = torch.empty(Bn, T, C, device="cuda")
    ctx.gemm_batched_f32(capi.OP_N, capi.OP_T, T, T, D, 1.0, Q, C, T * C, D, Kd, C, T * C, D, 0.0, S, T, H * T * T, T * T, Bn, H)
    ctx.causal_softmax_fwd_f32(S, S, scale, Bn * H * T, T)
    ctx.gemm_batched_f32(capi.OP_N, capi.OP_N, T, D, T, 1.0, S, T, H * T * T, T * T, Vd, C, T * C, D, 0.0, Oo, C, T * C, D, Bn, H)
    untok = lambda a: a.reshape(Bn, T, H, D).transpose(0, 2, 1, 3)
    assert max_abs_rel(untok(host(ctx, Oo)), o["attn.o"]) < TOL
    dP = torch.empty(Bn * H, T, T, device="cuda")
    dQ, dK, dV = torch.empty(Bn, T, C, device="cuda"), torch.empty(Bn, T, C, device="cuda"), torch.empty(Bn, T, C, device="cuda")
    ctx.gemm_batched_f32(capi.OP_T, capi.OP_N, T, D, T, 1.0, S, T, H * T * T, T * T, DO, C, T * C, D, 0.0, dV, C, T * C, D, Bn, H)
    ctx.gemm_batched_f32(capi.OP_N, capi.OP_T, T, T, D, 1.0, DO, C, T * C, D, Vd, C, T * C, D, 0.0, dP, T, H * T * T, T * T, Bn, H)
    ctx.causal_softmax_bwd_f32(dP, dP, S, scale, Bn * H * T, T, 0)
    ctx.gemm_batched_f32(capi.OP_N, capi.OP_N, T, D, T, 1.0, dP, T, H * T * T, T * T, Kd, C, T * C, D, 0.0, dQ, C, T * C, D, Bn, H)
    ctx.gemm_batched_f32(capi.OP_T, capi.OP_N, T, D, T, 1.0, dP, T, H * T * T, T * T, Q, C, T * C, D, 0.0, dK, C, T * C, D, Bn, H)
    assert max_abs_rel(untok(host(ctx, dQ)), o["attn.dq"]) < TOL
    assert max_abs_rel(untok(host(ctx, dK)), o["attn.dk"]) < TOL
    assert max_abs_rel(untok(host(ctx, dV)), o["attn.dv"]) < TOL


# ---- oracle parity on seeded inputs, fast-path shapes and ragged ones -------------------------------
@pytest.mark.parametrize("rows,cols", [(1, 128), (37, 256), (64, 768), (300, 1024), (5, 1000), (7, 2048), (3, 33), (0, 128)])
def test_layernorm_rmsnorm_vs_oracle(env, rows, cols):
    ctx, torch, capi = env
    x, dy = rnd(20, rows, cols) * 2 + 0.3, rnd(21, rows, cols, scale=1e-2)
    g, b = rnd(22, cols) * 0.2 + 1, rnd(23, cols) * 0.1
    X, DY, G, Bt = dev(torch, x), dev(torch, dy), dev(torch, g), dev(torch, b)
    y, s0, s1 = torch.empty(rows, cols, device="cuda"), torch.empty(max(rows, 1), device="cuda"), torch.empty(max(rows, 1), device="cuda")
    dx, dg, db = torch.ones(rows, cols, device="cuda"), torch.ones(cols, device="cuda"), torch.ones(cols, device="cuda")
    ctx.layernorm_fwd_f32(y, s0, s1, X, G, Bt, rows, cols, 1e-5)
    ctx.layernorm_bwd_f32(dx, dg, db, DY, X, G, s0, s1, rows, cols, 0, 0)
    if rows == 0:
        assert np.all(host(ctx, dg) == 0) and np.all(host(ctx, db) == 0)
        return
    ry, mu, rs = O.layernorm_fwd(x, g, b, 1e-5)
    rdx, rdg, rdb = O.layernorm_bwd(dy, x, g, mu, rs)
    assert max_abs_rel(host(ctx, y), ry) < TOL and max_abs_rel(host(ctx, dx), rdx) < TOL
    assert max_abs_rel(host(ctx, dg), rdg) < TOL and max_abs_rel(host(ctx, db), rdb) < TOL
    # accumulate flags
    ctx.layernorm_bwd_f32(dx, dg, db, DY, X, G, s0, s1, rows, cols, 1, 1)
    assert max_abs_rel(host(ctx, dx), 2 * rdx) < TOL and max_abs_rel(host(ctx, dg), 2 * rdg) < TOL
    ctx.rmsnorm_fwd_f32(y, s0, X, G, rows, cols, 1e-5)
    ctx.rmsnorm_bwd_f32(dx, dg, DY, X, G, s0, rows, cols, 0, 0)
    ry, inv = O.rmsnorm_fwd(x, g, 1e-5)
    rdx, rdg = O.rmsnorm_bwd(dy, x, g, inv)
    assert max_abs_rel(host(ctx, y), ry) < TOL and max_abs_rel(host(ctx, dx), rdx) < TOL and max_abs_rel(host(ctx, dg), rdg) < TOL


@pytest.mark.parametrize("rows,cols", [(8192, 1024), (5000, 768), (4736, 256), (6001, 512), (4800, 128)])
def test_norm_backward_staged_kernel_vs_oracle(env, rows, cols):
    """Row counts from 4 x 148 x 8 = 4736 up select the persistent kernel that stages rows through shared memory with bulk
    async copies (the LayerNorm / RMSNorm backward of every benchmarked shape).  It is held to the numpy oracle here with both
    accumulate flags, with dx left out, and with a row count that leaves the last sweep of the warps ragged."""
    ctx, torch, capi = env
    x, dy = rnd(120, rows, cols) * 2 + 0.3, rnd(121, rows, cols, scale=1e-2)
    g, b = rnd(122, cols) * 0.2 + 1, rnd(123, cols) * 0.1
    X, DY, G, Bt = dev(torch, x), dev(torch, dy), dev(torch, g), dev(torch, b)
    y, s0, s1 = torch.empty(rows, cols, device="cuda"), torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    # LayerNorm
    ctx.layernorm_fwd_f32(y, s0, s1, X, G, Bt, rows, cols, 1e-5)
    ry, mu, rs = O.layernorm_fwd(x, g, b, 1e-5)
    rdx, rdg, rdb = O.layernorm_bwd(dy, x, g, mu, rs)
    dx, dg, db = torch.full((rows, cols), 7.0, device="cuda"), torch.full((cols,), 7.0, device="cuda"), torch.full((cols,), 7.0, device="cuda")
    ctx.layernorm_bwd_f32(dx, dg, db, DY, X, G, s0, s1, rows, cols, 0, 0)
    assert max_abs_rel(host(ctx, y), ry) < TOL
    assert max_abs_rel(host(ctx, dx), rdx) < TOL and max_abs_rel(host(ctx, dg), rdg) < TOL and max_abs_rel(host(ctx, db), rdb) < TOL
    ctx.layernorm_bwd_f32(dx, dg, db, DY, X, G, s0, s1, rows, cols, 1, 0)   # dx accumulates, parameters overwrite
    assert max_abs_rel(host(ctx, dx), 2 * rdx) < TOL and max_abs_rel(host(ctx, dg), rdg) < TOL and max_abs_rel(host(ctx, db), rdb) < TOL
    ctx.layernorm_bwd_f32(dx, dg, db, DY, X, G, s0, s1, rows, cols, 0, 1)   # dx overwrites, parameters accumulate
    assert max_abs_rel(host(ctx, dx), rdx) < TOL and max_abs_rel(host(ctx, dg), 2 * rdg) < TOL and max_abs_rel(host(ctx, db), 2 * rdb) < TOL
    dg2, db2 = torch.full((cols,), 7.0, device="cuda"), torch.full((cols,), 7.0, device="cuda")
    ctx.layernorm_bwd_f32(None, dg2, db2, DY, X, G, s0, s1, rows, cols, 0, 0)  # parameter gradients only
    assert max_abs_rel(host(ctx, dg2), rdg) < TOL and max_abs_rel(host(ctx, db2), rdb) < TOL
    dx2 = torch.full((rows, cols), 7.0, device="cuda")
    ctx.layernorm_bwd_f32(dx2, None, None, DY, X, G, s0, s1, rows, cols, 0, 0)  # dx only
    assert max_abs_rel(host(ctx, dx2), rdx) < TOL
    # RMSNorm
    ctx.rmsnorm_fwd_f32(y, s0, X, G, rows, cols, 1e-5)
    ry, inv = O.rmsnorm_fwd(x, g, 1e-5)
    rdx, rdg = O.rmsnorm_bwd(dy, x, g, inv)
    dx.fill_(7.0); dg.fill_(7.0)
    ctx.rmsnorm_bwd_f32(dx, dg, DY, X, G, s0, rows, cols, 0, 0)
    assert max_abs_rel(host(ctx, y), ry) < TOL and max_abs_rel(host(ctx, dx), rdx) < TOL and max_abs_rel(host(ctx, dg), rdg) < TOL
    ctx.rmsnorm_bwd_f32(dx, dg, DY, X, G, s0, rows, cols, 1, 1)
    assert max_abs_rel(host(ctx, dx), 2 * rdx) < TOL and max_abs_rel(host(ctx, dg), 2 * rdg) < TOL
    ctx.rmsnorm_bwd_f32(None, dg, DY, X, G, s0, rows, cols, 0, 0)
    assert max_abs_rel(host(ctx, dg), rdg) < TOL


@pytest.mark.parametrize("rows", [4096, 16384])
def test_layernorm_bwd_is_deterministic(env, rows):
    ctx, torch, capi = env
    cols = 1024  # 4096 rows: warp-per-row kernel; 16384 rows: the staged persistent kernel
    x, dy, g = rnd(30, rows, cols), rnd(31, rows, cols, scale=1e-2), rnd(32, cols) + 1
    X, DY, G = dev(torch, x), dev(torch, dy), dev(torch, g)
    mu, rs = dev(torch, x.mean(1)), dev(torch, 1 / np.sqrt(x.var(1) + 1e-5))
    outs = []
    for _ in range(2):
        dx, dg, db = torch.empty(rows, cols, device="cuda"), torch.empty(cols, device="cuda"), torch.empty(cols, device="cuda")
        ctx.layernorm_bwd_f32(dx, dg, db, DY, X, G, mu, rs, rows, cols, 0, 0)
        outs.append((host(ctx, dx), host(ctx, dg), host(ctx, db)))
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("BH,T", [(3, 128), (2, 256), (2, 1024), (4, 20), (2, 33), (1, 1028)])
def test_causal_softmax_vs_oracle(env, BH, T):
    ctx, torch, capi = env
    s, dp = rnd(40, 1, BH, T, T) * 3, rnd(41, 1, BH, T, T, scale=1e-2)
    rows = BH * T
    P, dS = torch.empty(rows, T, device="cuda"), torch.full((rows, T), 7.0, device="cuda")
    ctx.causal_softmax_fwd_f32(P, dev(torch, s), 0.125, rows, T)
    rp = O.causal_softmax_fwd(s, 0.125)
    p = host(ctx, P).reshape(s.shape)
    assert max_abs_rel(p, rp) < TOL and np.all(np.triu(p, 1) == 0)
    assert np.allclose(p.sum(-1), 1.0, atol=1e-5)
    ctx.causal_softmax_bwd_f32(dS, dev(torch, dp), P, 0.125, rows, T, 0)
    rds = O.causal_softmax_bwd(dp, rp, 0.125)
    d = host(ctx, dS).reshape(s.shape)
    assert max_abs_rel(d, rds) < TOL and np.all(np.triu(d, 1) == 0)
    ctx.causal_softmax_bwd_f32(dS, dev(torch, dp), P, 0.125, rows, T, 1)
    assert max_abs_rel(host(ctx, dS).reshape(s.shape), 2 * rds) < TOL


@pytest.mark.parametrize("rows,V", [(5, 512), (33, 1000), (4, 32768), (2, 50257), (1, 7)])
def test_softmax_ce_vs_oracle(env, rows, V):
    ctx, torch, capi = env
    z = rnd(50, rows, V) * 3
    t = np.random.default_rng(51).integers(0, V, rows).astype(np.int32)
    Z, Tg = dev(torch, z), dev(torch, t)
    loss, P = torch.zeros(1, device="cuda"), torch.empty(rows, V, device="cuda")
    ctx.softmax_ce_fwd_f32(loss, P, Z, Tg, capi.IDX_I32, rows, V, 1e-5)
    rl, rp = O.softmax_ce_fwd(z, t.astype(np.int64), 1e-5)
    assert abs(float(host(ctx, loss)[0]) - float(rl)) / float(rl) < 1e-5
    assert max_abs_rel(host(ctx, P), rp) < TOL
    ctx.softmax_ce_bwd_f32(P, P, Tg, capi.IDX_I32, 1.0, rows, V, 0)
    rd = O.softmax_ce_bwd(rp, t.astype(np.int64), 1.0)
    d = host(ctx, P)
    assert max_abs_rel(d, rd) < TOL
    assert np.abs(d.sum(-1)).max() < 1e-6  # each row of dlogits sums to zero


def test_bad_targets_are_reported_not_dereferenced(env):
    ctx, torch, capi = env
    z = rnd(52, 4, 16)
    t = np.array([1, 99, 3, -1], dtype=np.int64)
    P, loss = torch.empty(4, 16, device="cuda"), torch.zeros(1, device="cuda")
    ctx.softmax_ce_fwd_f32(loss, P, dev(torch, z), dev(torch, t), capi.IDX_I64, 4, 16, 1e-5)
    with pytest.raises(capi.GcbError) as e:
        ctx.sync()
    assert e.value.status == capi.INVALID_ARG
    ctx.sync()  # the flag is cleared; the context stays usable


@pytest.mark.parametrize("n,V,W", [(64, 23, 12), (4096, 512, 128), (32768, 4096, 1024), (3000, 100, 36), (100, 10, 7), (5000, 50, 2052), (50000, 100003, 8), (33, 5, 4)])
def test_scatter_add_vs_oracle_and_determinism(env, n, V, W):
    ctx, torch, capi = env
    idx = synth.zipf_tokens(60, n, V)  # Zipf(1.1): heavy head rows
    dy = rnd(61, n, W, scale=1e-2)
    I, DY = dev(torch, idx), dev(torch, dy)
    base = rnd(62, V, W)
    runs = []
    for _ in range(2):
        d = dev(torch, base)
        ctx.scatter_add_f32(d, I, capi.IDX_I64, DY, n, W, V)
        runs.append(host(ctx, d))
    assert np.array_equal(runs[0], runs[1])  # no floating-point atomics: bitwise repeatable
    ref = O.scatter_add(base.astype(np.float64), idx, dy.astype(np.float64))
    assert max_abs_rel(runs[0], ref) < 1e-5
    untouched = np.bincount(idx, minlength=V) == 0
    assert np.array_equal(runs[0][untouched], base[untouched])
    order, counts, offsets = torch.empty(n, dtype=torch.int32, device="cuda"), torch.empty(V, dtype=torch.int32, device="cuda"), torch.empty(V + 1, dtype=torch.int32, device="cuda")
    ctx.scatter_plan_i32(order, counts, offsets, I, capi.IDX_I64, n, V)
    ro, rc, rf = O.scatter_plan(idx, V)
    assert np.array_equal(host(ctx, order), ro) and np.array_equal(host(ctx, counts), rc) and np.array_equal(host(ctx, offsets), rf)
    out = torch.empty(n, W, device="cuda")
    ctx.embed_f32(out, I, capi.IDX_I64, dev(torch, base), n, W, V)
    assert np.array_equal(host(ctx, out), base[idx])


@pytest.mark.parametrize("n", [1, 1023, 1024, 5000, 1 << 20])
def test_adamw_arena_matches_per_tensor(env, n):
    ctx, torch, capi = env
    w0, g = rnd(70, n, scale=0.02), rnd(71, n, scale=1e-2)
    chunks = (n + capi.ADAMW_CHUNK - 1) // capi.ADAMW_CHUNK
    mask = (np.arange(chunks) % 2).astype(np.uint8)
    w, m, v = dev(torch, w0), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    ctx.adamw_arena_f32(w, m, v, dev(torch, g), dev(torch, mask), n, 3e-4, 0.9, 0.95, 0.9, 0.95, 0.1, 1e-5, 0.5)
    decay = np.repeat(mask, capi.ADAMW_CHUNK)[:n].astype(bool)
    rw = np.empty_like(w0)
    for nd in (False, True):
        sel = decay != nd
        a, _, _ = O.adamw_step(w0[sel], g[sel] * np.float32(0.5), np.zeros(sel.sum(), np.float32), np.zeros(sel.sum(), np.float32), 3e-4, 0.9, 0.95, 0.9, 0.95, 0.1, 1e-5, nd)
        rw[sel] = a
    assert max_abs_rel(host(ctx, w), rw) < 1e-6


@pytest.mark.parametrize("opa,opb,M,N,K", [(0, 0, 65, 33, 17), (0, 1, 130, 257, 64), (1, 0, 96, 200, 300), (1, 1, 5, 7, 9), (0, 0, 256, 384, 512), (0, 0, 4, 8, 0)])
def test_gemm_simt_vs_numpy(env, opa, opb, M, N, K):
    ctx, torch, capi = env
    ctx.ctx_set_gemm_engine(1)
    try:
        A = rnd(80, *((K, M) if opa else (M, K)))
        Bm = rnd(81, *((N, K) if opb else (K, N)))
        C0, bias = rnd(82, M, N), rnd(83, N)
        C = dev(torch, C0)
        ctx.gemm_f32(opa, opb, M, N, K, 0.5, dev(torch, A), A.shape[1] if A.size else max(M, K, 1), dev(torch, Bm), Bm.shape[1] if Bm.size else max(N, K, 1), 2.0, C, N, dev(torch, bias))
        a = A.T if opa else A
        b = Bm.T if opb else Bm
        ref = 0.5 * (a.astype(np.float64) @ b.astype(np.float64)) + 2.0 * C0 + bias
        assert max_abs_rel(host(ctx, C), ref) < 1e-5
        assert ctx.ctx_last_gemm_engine() == 1
    finally:
        ctx.ctx_set_gemm_engine(0)


def test_arena_reuse_limit_and_errors(env):
    import ctypes

    ctx, torch, capi = env
    p1, p2 = ctypes.c_void_p(), ctypes.c_void_p()
    ctx.arena_alloc(1 << 20, ctypes.byref(p1))
    ctx.arena_alloc(1 << 20, ctypes.byref(p2))
    assert p1.value != p2.value and p1.value % 512 == 0
    used = ctx.arena_in_use_bytes()
    ctx.arena_free(p1)
    p3 = ctypes.c_void_p()
    ctx.arena_alloc(1 << 19, ctypes.byref(p3))
    assert p3.value == p1.value  # best fit reuses the freed block: no new device allocation
    ctx.arena_free(p2)
    ctx.arena_free(p3)
    assert ctx.arena_in_use_bytes() < used and ctx.arena_high_water_bytes() >= used
    with pytest.raises(capi.GcbError) as e:
        ctx.arena_free(ctypes.c_void_p(12345))
    assert e.value.status == capi.INVALID_ARG
    # simulated out-of-memory: a host-side limit, nothing is exhausted on the device
    ctx.arena_set_limit(ctx.arena_reserved_bytes() + (1 << 20))
    with pytest.raises(capi.GcbError) as e:
        ctx.arena_alloc(1 << 34, ctypes.byref(p1))
    assert e.value.status == capi.OOM
    ctx.arena_set_limit(0)
    with pytest.raises(capi.GcbError):
        ctx.gemm_f32(0, 0, 4, 4, 4, 1.0, None, 4, None, 4, 0.0, None, 4, None)


@pytest.mark.parametrize("T,band", [(256, 128), (1024, 128), (384, 128), (64, 128)])
def test_causal_softmax_band_variants(env, T, band):
    """Band-limited forms: identical on and below the diagonal and inside the diagonal block; nothing is written beyond it."""
    ctx, torch, capi = env
    BH = 2
    s, dp = rnd(90, 1, BH, T, T) * 3, rnd(91, 1, BH, T, T, scale=1e-2)
    rows = BH * T
    S = dev(torch, s)
    P = torch.full((rows, T), 5.0, device="cuda")
    ctx.causal_softmax_fwd_band_f32(P, S, 0.125, rows, T, band)
    p = host(ctx, P).reshape(BH, T, T)
    rp = O.causal_softmax_fwd(s, 0.125)[0]
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    inside = j < np.minimum(T, (i // band + 1) * band)
    assert max_abs_rel(np.where(inside, p, 0), np.where(inside, rp, 0)) < TOL
    assert np.all(p[:, ~inside] == 5.0)  # untouched
    Pfull = dev(torch, rp.reshape(rows, T))
    dS = torch.full((rows, T), 5.0, device="cuda")
    ctx.causal_softmax_bwd_band_f32(dS, dev(torch, dp), Pfull, 0.125, rows, T, 0, band)
    d = host(ctx, dS).reshape(BH, T, T)
    rd = O.causal_softmax_bwd(dp, rp[None], 0.125)[0]
    assert max_abs_rel(np.where(inside, d, 0), np.where(inside, rd, 0)) < TOL
    assert np.all(d[:, ~inside] == 5.0)


def test_bounded_wait_that_runs_out_is_reported_and_the_context_survives(env):
    """The failure path of every barrier wait: a wait that nothing completes gives up after its poll budget (~10 ms here),
    the kernel returns normally, sync reports GCB_TIMEOUT once, and the same context keeps computing."""
    ctx, torch, capi = env
    ctx.selftest_bounded_wait(512)
    with pytest.raises(capi.GcbError) as e:
        ctx.sync()
    assert e.value.status == capi.TIMEOUT
    x = torch.empty(1000, device="cuda")
    ctx.fill_f32(x, 2.5, 1000)
    ctx.sync()  # the status word was cleared
    assert float(x.sum()) == 2500.0
