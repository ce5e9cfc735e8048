"""Seeded synthetic weights and token streams shared by the tests, the CPU checker and the bench.

Stands in for the reference's tokenised training file (README.md:110 of the reference); the
values are regenerated identically everywhere from a counter-based generator:
u = top 53 bits of splitmix64(seed * GOLDEN + index) / 2**53.
"""
import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _mix(z):
    with np.errstate(over="ignore"):
        z = (z + _GOLDEN).astype(np.uint64)
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform53(seed, n, start=0):
    """n doubles in [0, 1): element i depends only on (seed, start + i)."""
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + n, dtype=np.uint64)
        base = _mix(np.full(1, np.uint64(seed), dtype=np.uint64))[0]
        bits = _mix(base + idx * _GOLDEN)
    return (bits >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def name_seed(seed, name):
    """FNV-1a of the parameter name folded with the run seed: one independent stream per tensor."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return (h ^ (seed * 0x9E3779B97F4A7C15)) & 0xFFFFFFFFFFFFFFFF


def normal(seed, name, shape, std, mean=0.0):
    n = int(np.prod(shape)) if len(shape) else 1
    m = (n + 1) // 2
    u = uniform53(name_seed(seed, name), 2 * m)
    u1 = 1.0 - u[:m]  # (0, 1]
    u2 = u[m:]
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.concatenate([r * np.cos(2 * np.pi * u2), r * np.sin(2 * np.pi * u2)])[:n]
    return (mean + std * z).astype(np.float32).reshape(shape)


def zipf_cdf(vocab, s=1.1):
    w = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    c = np.cumsum(w)
    return c / c[-1]


def zipf_tokens(seed, count, vocab, s=1.1, start=0):
    """count token ids drawn i.i.d. from p(k) ~ (k+1)^-s over [0, vocab) by inverse CDF."""
    u = uniform53(seed, count, start)
    t = np.searchsorted(zipf_cdf(vocab, s), u, side="right")
    return np.minimum(t, vocab - 1).astype(np.int64)


def token_batches(seed, n_batches, B, T, vocab, s=1.1):
    """[n_batches, 2, B, T] int64: inputs and shift-by-one targets (data_loader.hpp:81-84 of the reference)."""
    out = np.empty((n_batches, 2, B, T), dtype=np.int64)
    per = B * (T + 1)
    for i in range(n_batches):
        t = zipf_tokens(seed, per, vocab, s, start=i * per).reshape(B, T + 1)
        out[i, 0] = t[:, :T]
        out[i, 1] = t[:, 1:]
    return out


def gpt_param_shapes(arch, V, T, C, H, L, F):
    """Ordered {name: (shape, kind)} with kind in {'matrix','bias','gamma','beta'}; names follow Module::register_*."""
    p = {}
    p["token_embed.embeds"] = ((V, C), "matrix")
    p["pos_embed.pos_embeds"] = ((T, C), "matrix")
    for i in range(L):
        b = "block_%d." % i
        p[b + "norm1.gamma"] = ((C,), "gamma")
        if arch == "lngelu":
            p[b + "norm1.beta"] = ((C,), "beta")
        for q in ("q_proj", "k_proj", "v_proj", "out_proj"):
            p[b + "attn." + q + ".W"] = ((C, C), "matrix")
            p[b + "attn." + q + ".b"] = ((C,), "bias")
        p[b + "norm2.gamma"] = ((C,), "gamma")
        if arch == "lngelu":
            p[b + "norm2.beta"] = ((C,), "beta")
            p[b + "mlp.fc1.W"] = ((C, F), "matrix")
            p[b + "mlp.fc1.b"] = ((F,), "bias")
            p[b + "mlp.fc2.W"] = ((F, C), "matrix")
            p[b + "mlp.fc2.b"] = ((C,), "bias")
        else:
            for w in ("w1", "w2"):
                p[b + "mlp." + w + ".W"] = ((C, 3 * C), "matrix")
                p[b + "mlp." + w + ".b"] = ((3 * C,), "bias")
            p[b + "mlp.w3.W"] = ((3 * C, C), "matrix")
            p[b + "mlp.w3.b"] = ((C,), "bias")
    p["final_norm.gamma"] = ((C,), "gamma")
    if arch == "lngelu":
        p["final_norm.beta"] = ((C,), "beta")
    return p


def gpt_weights(arch, V, T, C, H, L, F, seed=0, std=0.02, perturb=False):
    """Seeded weights: matrices N(0, std), biases 0, gamma 1, beta 0.

    perturb=True draws biases/gamma/beta around their defaults as well, so that parity tests
    exercise every gradient path with non-trivial values.
    """
    w = {}
    for name, (shape, kind) in gpt_param_shapes(arch, V, T, C, H, L, F).items():
        if kind == "matrix":
            w[name] = normal(seed, name, shape, std)
        elif kind == "gamma":
            w[name] = normal(seed, name, shape, 0.1, 1.0) if perturb else np.ones(shape, np.float32)
        else:
            w[name] = normal(seed, name, shape, 0.05) if perturb else np.zeros(shape, np.float32)
    return w
