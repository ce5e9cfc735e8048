"""gcb_layernorm_bwd_noalloc_f32: the LayerNorm backward for callers that may not allocate (a host thread that must never
block on an allocator lock, or an embedding application that owns all device memory).  It keeps its scratch in a fixed
device array inside the library instead of taking a block from the context's arena.

Checked here, through the C ABI: it gives the same dx / dgamma / dbeta as gcb_layernorm_bwd_f32 and as the numpy oracle on
two calls in a row with different inputs and sizes (the shared array keeps the previous call's contents, which must not leak into the next
result), it leaves the arena untouched, and it refuses sizes its array cannot hold.  This file sorts last so that a run
stopping at the first failure has already executed every other test."""
import numpy as np
import pytest

from oracle import numpy_oracle as O
from tests.helpers import max_abs_rel

pytestmark = pytest.mark.gpu
TOL = 1e-4  # the tolerance of the other kernel tests; the two entry points share their kernels, so they normally agree exactly


def test_noalloc_layernorm_bwd_matches_arena_version_twice():
    import torch

    from gradcraft_b200 import capi

    ctx = capi.Context(0)
    try:
        for call, (rows, cols) in enumerate([(3000, 1024), (517, 256)]):
            rng = np.random.default_rng(100 + call)
            x = rng.standard_normal((rows, cols), dtype=np.float32) * 2 + 0.5
            dy = rng.standard_normal((rows, cols), dtype=np.float32) * 1e-2
            g = (1 + 0.2 * rng.standard_normal(cols, dtype=np.float32)).astype(np.float32)
            b = np.zeros(cols, np.float32)
            X, DY, G, Bt = (torch.from_numpy(a).cuda() for a in (x, dy, g, b))
            y, mu, rs = torch.empty(rows, cols, device="cuda"), torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
            ctx.layernorm_fwd_f32(y, mu, rs, X, G, Bt, rows, cols, 1e-5)
            ref = [torch.empty(rows, cols, device="cuda"), torch.empty(cols, device="cuda"), torch.empty(cols, device="cuda")]
            ctx.layernorm_bwd_f32(ref[0], ref[1], ref[2], DY, X, G, mu, rs, rows, cols, 0, 0)
            ctx.sync()
            in_use, reserved, hwm = ctx.arena_in_use_bytes(), ctx.arena_reserved_bytes(), ctx.arena_high_water_bytes()
            got = [torch.full((rows, cols), 3.0, device="cuda"), torch.full((cols,), 3.0, device="cuda"), torch.full((cols,), 3.0, device="cuda")]
            ctx.layernorm_bwd_noalloc_f32(got[0], got[1], got[2], DY, X, G, mu, rs, rows, cols, 0, 0)
            ctx.sync()
            assert (ctx.arena_in_use_bytes(), ctx.arena_reserved_bytes(), ctx.arena_high_water_bytes()) == (in_use, reserved, hwm)
            for a, r in zip(got, ref):
                assert max_abs_rel(a.cpu().numpy(), r.cpu().numpy()) < TOL
            # and the independent checker: the numpy restatement of the reference's LayerNorm backward
            _, o_mu, o_rs = O.layernorm_fwd(x, g, b, 1e-5)
            for a, r in zip(got, O.layernorm_bwd(dy, x, g, o_mu, o_rs)):
                assert max_abs_rel(a.cpu().numpy(), r) < TOL
            # accumulate flags behave the same way
            ctx.layernorm_bwd_noalloc_f32(got[0], got[1], got[2], DY, X, G, mu, rs, rows, cols, 1, 1)
            ctx.sync()
            for a, r in zip(got, ref):
                assert max_abs_rel(a.cpu().numpy(), 2 * r.cpu().numpy()) < TOL
        # beyond the fixed array: a clear refusal, not a silent fallback
        big = torch.zeros(4, 2048, device="cuda")
        v = torch.zeros(2048, device="cuda")
        s = torch.zeros(4, device="cuda")
        with pytest.raises(capi.GcbError) as e:
            ctx.layernorm_bwd_noalloc_f32(big, v, v, big, big, v, s, s, 4, 2048, 0, 0)
        assert e.value.status == capi.INVALID_ARG and "1024" in str(e.value)
    finally:
        ctx.close()
