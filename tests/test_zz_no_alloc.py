"""lcu_rope_scatter_static - the RoPE + cache-write operator that allocates nothing - must give
exactly what lcu_rope_scatter gives.  It exists for callers that cannot call cudaMalloc (all of HBM
already owned by their own pool, or no tolerance for cudaMalloc's device-wide synchronisation), so
its cos/sin table sits in a fixed device array inside the library.  The array is shared by all calls
and keeps the last call's contents; two different calls in a row check that stale contents do no harm.
Collected last on purpose: a failure here cannot hide the other tests' results."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run(lcu, fn, q, k, v, n_heads, pos0, ctx):
    m, dim = q.shape
    dq, dk, dv = lcu.DeviceBuffer.from_host(q), lcu.DeviceBuffer.from_host(k), lcu.DeviceBuffer.from_host(v)
    kc, vc = lcu.DeviceBuffer(ctx * dim * 2), lcu.DeviceBuffer(ctx * dim * 2)
    lcu.check(lcu.lib.lcu_memset(kc.ptr, 0, kc.nbytes))
    lcu.check(lcu.lib.lcu_memset(vc.ptr, 0, vc.nbytes))
    lcu.check(fn(dq.ptr, dk.ptr, dv.ptr, kc.ptr, vc.ptr, pos0, m, dim, n_heads, ctx, None))
    lcu.check(lcu.lib.lcu_synchronize())
    return dq.to_host(np.uint16, (m, dim)), kc.to_host(np.uint16, (ctx * dim,)), vc.to_host(np.uint16, (ctx * dim,))


def test_static_variant_equals_allocating_variant_twice_in_a_row(lcu):
    rng = np.random.default_rng(42)
    # second call: other head_dim and positions, so the table left by the first call is stale everywhere it is reused
    for m, dim, n_heads, pos0, ctx in ((5, 256, 2, 9, 64), (3, 256, 4, 40, 48)):
        q, k, v = (rng.standard_normal((m, dim)).astype(np.float16).view(np.uint16) for _ in range(3))
        want = run(lcu, lcu.lib.lcu_rope_scatter, q, k, v, n_heads, pos0, ctx)
        got = run(lcu, lcu.lib.lcu_rope_scatter_static, q, k, v, n_heads, pos0, ctx)
        for a, b in zip(got, want):
            assert (a == b).all()  # same kernels, same table values: bit identical


def test_static_variant_rejects_requests_beyond_its_table(lcu):
    d = lcu.DeviceBuffer(1 << 12)
    rc = lcu.lib.lcu_rope_scatter_static(d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, 4096, 1, 256, 2, 8192, None)
    assert rc == 2 and b"exceed the static table" in lcu.lib.lcu_last_error()
