"""numpy restatement of the GradCraft training hot path in fp32 (test infrastructure only).

Pinned against outputs of the compiled reference CPU path (oracle/_ref, fixtures under
tests/golden/): the reference ships no tests or golden vectors of its own.
File:line citations are paths inside the reference project.
"""
import numpy as np

F32 = np.float32
GELU_A = F32(0.7978845608)  # backend/cuda/math_functors.cuh:428
GELU_B = F32(0.044715)


# ---- normalisation -------------------------------------------------------------------------------
def layernorm_fwd(x, gamma, beta, eps):
    """graph/nodes/normalization_nodes.hpp:24-82: biased variance, eps inside the sqrt."""
    x = x.astype(F32)
    mu = x.mean(axis=-1, keepdims=True, dtype=F32)
    xc = x - mu
    var = (xc * xc).mean(axis=-1, keepdims=True, dtype=F32)
    rstd = F32(1.0) / np.sqrt(var + F32(eps))
    xhat = xc * rstd
    return xhat * gamma + beta, mu[..., 0], rstd[..., 0]


def layernorm_bwd(dy, x, gamma, mu, rstd):
    """normalization_nodes.hpp:84-134: dbeta=sum dy, dgamma=sum dy*xhat, dx=rstd*(g-mean(g)-xhat*mean(g*xhat))."""
    xhat = (x - mu[..., None]) * rstd[..., None]
    red = tuple(range(dy.ndim - 1))
    dbeta = dy.sum(axis=red, dtype=np.float64).astype(F32)
    dgamma = (dy * xhat).sum(axis=red, dtype=np.float64).astype(F32)
    g = dy * gamma
    m1 = g.mean(axis=-1, keepdims=True, dtype=F32)
    m2 = (g * xhat).mean(axis=-1, keepdims=True, dtype=F32)
    dx = (g - m1 - xhat * m2) * rstd[..., None]
    return dx.astype(F32), dgamma, dbeta


def rmsnorm_fwd(x, gamma, eps):
    """backend/cuda/kernels_math.cu:787-838: inv = 1/sqrt(mean(x^2)+eps); y = x*inv*gamma."""
    inv = F32(1.0) / np.sqrt((x * x).mean(axis=-1, keepdims=True, dtype=F32) + F32(eps))
    return (x * inv * gamma).astype(F32), inv[..., 0].astype(F32)


def rmsnorm_bwd(dy, x, gamma, inv):
    """kernels_math.cu:977-1043: s = mean(dy*gamma*xhat); dx = inv*(dy*gamma - xhat*s); dgamma = sum dy*xhat."""
    xhat = x * inv[..., None]
    g = dy * gamma
    s = (g * xhat).mean(axis=-1, keepdims=True, dtype=F32)
    dx = inv[..., None] * (g - xhat * s)
    red = tuple(range(dy.ndim - 1))
    dgamma = (dy * xhat).sum(axis=red, dtype=np.float64).astype(F32)
    return dx.astype(F32), dgamma


# ---- activations ---------------------------------------------------------------------------------
def gelu_fwd(x):
    """tanh approximation, math_functors.cuh:425-443."""
    return (x * F32(0.5) * (F32(1.0) + np.tanh(GELU_A * (x + GELU_B * x * x * x)))).astype(F32)


def gelu_bwd(dy, x):
    """BGeLU, math_functors.cuh:184-214."""
    x2 = x * x
    t = np.tanh(GELU_A * (x + GELU_B * x2 * x))
    up = GELU_A * (F32(1.0) + F32(3.0) * GELU_B * x2)
    local = F32(0.5) * (F32(1.0) + t) + F32(0.5) * x * (F32(1.0) - t * t) * up
    return (dy * local).astype(F32)


def _sigmoid(a):
    return F32(1.0) / (F32(1.0) + np.exp(-a))


def swiglu_fwd(a, b):
    """kernels_math.cu:1507-1524: silu(a) * b."""
    return (a * _sigmoid(a) * b).astype(F32)


def swiglu_bwd(dy, a, b):
    """kernels_math.cu:1543-1579: da = g*b*sig*(1+a*(1-sig)); db = g*silu(a)."""
    s = _sigmoid(a)
    da = dy * b * s * (F32(1.0) + a * (F32(1.0) - s))
    db = dy * a * s
    return da.astype(F32), db.astype(F32)


# ---- attention softmax ---------------------------------------------------------------------------
def causal_softmax_fwd(scores, scale):
    """kernels_math.cu:1204-1271: softmax over j<=i of scores*scale, exact zeros above the diagonal."""
    T = scores.shape[-1]
    keep = np.tril(np.ones((T, T), dtype=bool))
    s = np.where(keep, scores * F32(scale), -np.inf).astype(F32)
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    return (e / e.sum(axis=-1, keepdims=True, dtype=F32)).astype(F32)


def causal_softmax_bwd(dp, probs, scale):
    """kernels_math.cu:1287-1337: dS = scale * P * (dP - sum_j dP_j P_j), zero above the diagonal."""
    dot = (dp * probs).sum(axis=-1, keepdims=True, dtype=F32)
    return (F32(scale) * probs * (dp - dot)).astype(F32)


# ---- loss ----------------------------------------------------------------------------------------
def softmax_ce_fwd(logits, targets, eps):
    """kernels_math.cu:1357-1426 / loss_nodes.hpp:24-60: probs, loss = mean(-log(p_t + eps))."""
    z = logits.astype(F32)
    m = z.max(axis=-1, keepdims=True)
    e = np.exp(z - m)
    p = (e / e.sum(axis=-1, keepdims=True, dtype=F32)).astype(F32)
    rows = p.shape[0]
    pt = p[np.arange(rows), targets]
    loss = F32((-np.log(pt + F32(eps))).astype(np.float64).sum() / rows)
    return loss, p


def softmax_ce_bwd(probs, targets, upstream):
    """kernels_math.cu:1449-1482: dx = (p - onehot) * upstream / rows (eps ignored)."""
    rows = probs.shape[0]
    s = F32(upstream) / F32(rows)
    d = probs * s
    d[np.arange(rows), targets] -= s
    return d.astype(F32)


# ---- embedding -----------------------------------------------------------------------------------
def embed_fwd(idx, table):
    """kernels_math.cu:581-595: row gather."""
    return table[idx]


def scatter_add(dtable, idx, dy):
    """backend/cpu/apply.hpp:464-529: dE[idx[i], :] += dy[i, :], visiting i in ascending order."""
    flat = idx.reshape(-1)
    d2 = dy.reshape(flat.size, -1)
    np.add.at(dtable, flat, d2)
    return dtable


def scatter_plan(idx, vocab):
    """Integer bookkeeping of a sorted scatter-add: stable order of positions by row, per-row hit
    counts and exclusive segment offsets.  Compared bit-exactly with the device plan."""
    flat = idx.reshape(-1).astype(np.int64)
    order = np.argsort(flat, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=vocab).astype(np.int32)
    offsets = np.zeros(vocab + 1, dtype=np.int32)
    np.cumsum(counts, out=offsets[1:])
    return order, counts, offsets


# ---- linear / attention --------------------------------------------------------------------------
def linear_fwd(x, W, b):
    """nn/layers/linear.hpp:22-25: y = x.W + b with W (in, out)."""
    return (x.reshape(-1, W.shape[0]) @ W + b).reshape(*x.shape[:-1], W.shape[1]).astype(F32)


def linear_bwd(dy, x, W):
    """graph/nodes/math_nodes.hpp:505-530: dX = dY.W^T, dW = X^T.dY; bias grad = column sums."""
    d2 = dy.reshape(-1, W.shape[1])
    x2 = x.reshape(-1, W.shape[0])
    return (d2 @ W.T).reshape(x.shape).astype(F32), (x2.T @ d2).astype(F32), d2.sum(axis=0, dtype=np.float64).astype(F32)


def attention_fwd(q, k, v):
    """frontend/tensor_other.hpp:53-93 on (B,H,T,D): P = causal_softmax(q k^T / sqrt(D)); O = P v."""
    scale = F32(1.0 / np.sqrt(q.shape[-1]))
    p = causal_softmax_fwd(q @ k.transpose(0, 1, 3, 2), scale)
    return (p @ v).astype(F32), p


def attention_bwd(do, q, k, v, p):
    scale = F32(1.0 / np.sqrt(q.shape[-1]))
    dv = p.transpose(0, 1, 3, 2) @ do
    dp = do @ v.transpose(0, 1, 3, 2)
    ds = causal_softmax_bwd(dp, p, scale)
    dq = ds @ k
    dk = ds.transpose(0, 1, 3, 2) @ q
    return dq.astype(F32), dk.astype(F32), dv.astype(F32)


# ---- optimizer -----------------------------------------------------------------------------------
def global_norm_clip(grads, max_norm):
    """nn/utils/norm_clip.hpp:15-58: n = sqrt(sum g^2); if n > max: g *= max / (n + 1e-6)."""
    sq = F32(0)
    for g in grads.values():
        sq = F32(sq + F32((g.astype(F32) ** 2).sum(dtype=np.float64)))
    n = F32(np.sqrt(sq))
    if n > F32(max_norm):
        s = F32(max_norm) / (n + F32(1e-6))
        for k in grads:
            grads[k] = (grads[k] * s).astype(F32)
    return n


def adamw_step(w, g, m, v, lr, beta1, beta2, beta1_exp, beta2_exp, wd, eps, no_decay):
    """kernels_math.cu:1604-1646.  beta*_exp are beta^t already advanced for this step (adam.hpp:44-45)."""
    lr, beta1, beta2, wd, eps = F32(lr), F32(beta1), F32(beta2), F32(wd), F32(eps)
    if not no_decay:
        w = w * (F32(1.0) - lr * wd)
    m = beta1 * m + (F32(1.0) - beta1) * g
    v = beta2 * v + (F32(1.0) - beta2) * g * g
    mh = m / (F32(1.0) - F32(beta1_exp))
    vh = v / (F32(1.0) - F32(beta2_exp))
    w = w - lr * mh / (np.sqrt(vh) + eps)
    return w.astype(F32), m.astype(F32), v.astype(F32)


def cosine_lr(t, max_lr, min_lr, warmup, total):
    """nn/sched/cosine_scheduler.hpp:20-36 with t already incremented."""
    if t <= warmup:
        return F32(max_lr) * (F32(t) / F32(warmup))
    if t >= total:
        return F32(min_lr)
    r = F32(t - warmup) / F32(total - warmup)
    c = F32(0.5) * (F32(1.0) + np.cos(F32(np.pi) * r, dtype=F32))
    return F32(min_lr) + c * (F32(max_lr) - F32(min_lr))


NO_DECAY_SUFFIXES = (".b", ".gamma", ".beta", ".embeds", ".pos_embeds")  # linear.hpp:16, normalization.hpp:41, other.hpp:16,41


def is_no_decay(name):
    return name.endswith(NO_DECAY_SUFFIXES)


# ---- whole model ---------------------------------------------------------------------------------
class GPTOracle:
    """fwd + bwd of the transformer as the reference assembles it (nn/layers/gpt.hpp:41-112,
    attention.hpp:44-73); arch 'lngelu' swaps RMSNorm/SwiGLU for LayerNorm/GELU with d_ff = F."""

    def __init__(self, arch, V, T, C, H, L, F, norm_eps=1e-5, ce_eps=1e-5):
        self.arch, self.V, self.T, self.C, self.H, self.L, self.F = arch, V, T, C, H, L, F
        self.norm_eps, self.ce_eps = norm_eps, ce_eps

    def _norm_f(self, w, pre, x):
        if self.arch == "lngelu":
            y, mu, rstd = layernorm_fwd(x, w[pre + ".gamma"], w[pre + ".beta"], self.norm_eps)
            return y, (x, mu, rstd)
        y, inv = rmsnorm_fwd(x, w[pre + ".gamma"], self.norm_eps)
        return y, (x, inv)

    def _norm_b(self, w, g, pre, dy, cache):
        if self.arch == "lngelu":
            x, mu, rstd = cache
            dx, dg, db = layernorm_bwd(dy, x, w[pre + ".gamma"], mu, rstd)
            g[pre + ".gamma"] = dg
            g[pre + ".beta"] = db
            return dx
        x, inv = cache
        dx, dg = rmsnorm_bwd(dy, x, w[pre + ".gamma"], inv)
        g[pre + ".gamma"] = dg
        return dx

    def logits(self, w, X):
        """Forward only: (B, T, V) logits of the tied head (the forward half of loss_and_grads; nn/layers/gpt.hpp:99-110)."""
        B, T = X.shape
        C, H = self.C, self.H
        D = C // H
        x = (w["token_embed.embeds"][X] + w["pos_embed.pos_embeds"][:T][None]).astype(F32)
        split = lambda t: t.reshape(B, T, H, D).transpose(0, 2, 1, 3)
        for i in range(self.L):
            b = "block_%d." % i
            h1, _ = self._norm_f(w, b + "norm1", x)
            q, k, v = (linear_fwd(h1, w[b + "attn.%s_proj.W" % n], w[b + "attn.%s_proj.b" % n]) for n in "qkv")
            o, _ = attention_fwd(split(q), split(k), split(v))
            x = x + linear_fwd(o.transpose(0, 2, 1, 3).reshape(B, T, C), w[b + "attn.out_proj.W"], w[b + "attn.out_proj.b"])
            h2, _ = self._norm_f(w, b + "norm2", x)
            if self.arch == "lngelu":
                x = x + linear_fwd(gelu_fwd(linear_fwd(h2, w[b + "mlp.fc1.W"], w[b + "mlp.fc1.b"])), w[b + "mlp.fc2.W"], w[b + "mlp.fc2.b"])
            else:
                u1 = linear_fwd(h2, w[b + "mlp.w1.W"], w[b + "mlp.w1.b"])
                u2 = linear_fwd(h2, w[b + "mlp.w2.W"], w[b + "mlp.w2.b"])
                x = x + linear_fwd(swiglu_fwd(u1, u2), w[b + "mlp.w3.W"], w[b + "mlp.w3.b"])
        xf, _ = self._norm_f(w, "final_norm", x)
        return (xf.reshape(B * T, C) @ w["token_embed.embeds"].T).astype(F32).reshape(B, T, -1)

    def loss_and_grads(self, w, X, Y, upstream=1.0):
        B, T = X.shape
        C, H = self.C, self.H
        D = C // H
        tape = []
        x = (w["token_embed.embeds"][X] + w["pos_embed.pos_embeds"][:T][None]).astype(F32)
        for i in range(self.L):
            b = "block_%d." % i
            c = {}
            h1, c["n1"] = self._norm_f(w, b + "norm1", x)
            c["h1"] = h1
            q = linear_fwd(h1, w[b + "attn.q_proj.W"], w[b + "attn.q_proj.b"])
            k = linear_fwd(h1, w[b + "attn.k_proj.W"], w[b + "attn.k_proj.b"])
            v = linear_fwd(h1, w[b + "attn.v_proj.W"], w[b + "attn.v_proj.b"])
            split = lambda t: t.reshape(B, T, H, D).transpose(0, 2, 1, 3)
            c["q"], c["k"], c["v"] = split(q), split(k), split(v)
            o, c["p"] = attention_fwd(c["q"], c["k"], c["v"])
            c["a"] = o.transpose(0, 2, 1, 3).reshape(B, T, C)
            x = x + linear_fwd(c["a"], w[b + "attn.out_proj.W"], w[b + "attn.out_proj.b"])
            h2, c["n2"] = self._norm_f(w, b + "norm2", x)
            c["h2"] = h2
            if self.arch == "lngelu":
                c["u"] = linear_fwd(h2, w[b + "mlp.fc1.W"], w[b + "mlp.fc1.b"])
                c["gu"] = gelu_fwd(c["u"])
                x = x + linear_fwd(c["gu"], w[b + "mlp.fc2.W"], w[b + "mlp.fc2.b"])
            else:
                c["u1"] = linear_fwd(h2, w[b + "mlp.w1.W"], w[b + "mlp.w1.b"])
                c["u2"] = linear_fwd(h2, w[b + "mlp.w2.W"], w[b + "mlp.w2.b"])
                c["s"] = swiglu_fwd(c["u1"], c["u2"])
                x = x + linear_fwd(c["s"], w[b + "mlp.w3.W"], w[b + "mlp.w3.b"])
            tape.append(c)
        xf, nf = self._norm_f(w, "final_norm", x)
        E = w["token_embed.embeds"]
        logits = (xf.reshape(B * T, C) @ E.T).astype(F32)
        loss, probs = softmax_ce_fwd(logits, Y.reshape(-1), self.ce_eps)

        g = {}
        dlog = softmax_ce_bwd(probs, Y.reshape(-1), upstream)
        dE = (dlog.T @ xf.reshape(B * T, C)).astype(F32)  # tied head contribution
        dx = self._norm_b(w, g, "final_norm", (dlog @ E).reshape(B, T, C).astype(F32), nf)
        merge = lambda t: t.transpose(0, 2, 1, 3).reshape(B, T, C)
        for i in reversed(range(self.L)):
            b = "block_%d." % i
            c = tape[i]
            if self.arch == "lngelu":
                dgu, g[b + "mlp.fc2.W"], g[b + "mlp.fc2.b"] = linear_bwd(dx, c["gu"], w[b + "mlp.fc2.W"])
                du = gelu_bwd(dgu, c["u"])
                dh2, g[b + "mlp.fc1.W"], g[b + "mlp.fc1.b"] = linear_bwd(du, c["h2"], w[b + "mlp.fc1.W"])
            else:
                ds, g[b + "mlp.w3.W"], g[b + "mlp.w3.b"] = linear_bwd(dx, c["s"], w[b + "mlp.w3.W"])
                du1, du2 = swiglu_bwd(ds, c["u1"], c["u2"])
                dh2a, g[b + "mlp.w2.W"], g[b + "mlp.w2.b"] = linear_bwd(du2, c["h2"], w[b + "mlp.w2.W"])
                dh2b, g[b + "mlp.w1.W"], g[b + "mlp.w1.b"] = linear_bwd(du1, c["h2"], w[b + "mlp.w1.W"])
                dh2 = dh2a + dh2b
            dx = dx + self._norm_b(w, g, b + "norm2", dh2, c["n2"])
            da, g[b + "attn.out_proj.W"], g[b + "attn.out_proj.b"] = linear_bwd(dx, c["a"], w[b + "attn.out_proj.W"])
            do = da.reshape(B, T, H, D).transpose(0, 2, 1, 3)
            dq, dk, dv = attention_bwd(do, c["q"], c["k"], c["v"], c["p"])
            dh1v, g[b + "attn.v_proj.W"], g[b + "attn.v_proj.b"] = linear_bwd(merge(dv), c["h1"], w[b + "attn.v_proj.W"])
            dh1k, g[b + "attn.k_proj.W"], g[b + "attn.k_proj.b"] = linear_bwd(merge(dk), c["h1"], w[b + "attn.k_proj.W"])
            dh1q, g[b + "attn.q_proj.W"], g[b + "attn.q_proj.b"] = linear_bwd(merge(dq), c["h1"], w[b + "attn.q_proj.W"])
            dx = dx + self._norm_b(w, g, b + "norm1", dh1v + dh1k + dh1q, c["n1"])
        pos = np.zeros_like(w["pos_embed.pos_embeds"])
        pos[:T] = dx.sum(axis=0, dtype=np.float64).astype(F32)
        g["pos_embed.pos_embeds"] = pos
        g["token_embed.embeds"] = scatter_add(dE, X, dx)
        return loss, g

    def train(self, w, batches, steps, accum, lr, beta1, beta2, wd, eps, clip=0.0, record=(1,)):
        """batches: [steps*accum, 2, B, T].  Returns losses, {step: grads}, {step: weights}."""
        w = {k: v.copy() for k, v in w.items()}
        m = {k: np.zeros_like(v) for k, v in w.items()}
        v2 = {k: np.zeros_like(v) for k, v in w.items()}
        b1e, b2e = F32(1.0), F32(1.0)
        losses, grads_at, weights_at = [], {}, {}
        for step in range(1, steps + 1):
            grads, tot = None, 0.0
            for mb in range(accum):
                X, Y = batches[(step - 1) * accum + mb]
                loss, g = self.loss_and_grads(w, X, Y, upstream=1.0 / accum)
                tot += float(loss) / accum
                grads = g if grads is None else {k: grads[k] + g[k] for k in g}
            if step in record:
                grads_at[step] = {k: a.copy() for k, a in grads.items()}
            if clip > 0:
                global_norm_clip(grads, clip)
            b1e, b2e = F32(b1e * F32(beta1)), F32(b2e * F32(beta2))
            for k in w:
                w[k], m[k], v2[k] = adamw_step(w[k], grads[k], m[k], v2[k], lr, beta1, beta2, b1e, b2e, wd, eps, is_no_decay(k))
            losses.append(tot)
            if step in record:
                weights_at[step] = {k: a.copy() for k, a in w.items()}
        return losses, grads_at, weights_at
