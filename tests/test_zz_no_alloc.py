"""lcu_rope_scatter_static - the RoPE + cache-write operator that allocates nothing - must give
exactly what lcu_rope_scatter gives.  It exists for callers that cannot call cudaMalloc (all of HBM
already owned by their own pool, or no tolerance for cudaMalloc's device-wide synchronisation), so
its cos/sin table sits in a fixed device array inside the library.  The array is shared by all calls
and keeps the last call's contents; two different calls in a row check that stale contents do no harm.
The first call on a device is the one that makes the CUDA runtime load the module holding the array
(2 MiB); after it, calls must not change the amount of free device memory.
Collected last on purpose: a failure here cannot hide the other tests' results."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu


def f32(u):
    return np.asarray(u, np.uint16).view(np.float16).astype(np.float32)


def run(lcu, fn, q, k, v, n_heads, pos0, ctx, bufs=None):
    m, dim = q.shape
    if bufs is None:
        bufs = [lcu.DeviceBuffer(q.nbytes), lcu.DeviceBuffer(k.nbytes), lcu.DeviceBuffer(v.nbytes), lcu.DeviceBuffer(ctx * dim * 2),
                lcu.DeviceBuffer(ctx * dim * 2)]
    dq, dk, dv, kc, vc = bufs
    for d, a in ((dq, q), (dk, k), (dv, v)):
        lcu.check(lcu.lib.lcu_memcpy_h2d(d.ptr, a.ctypes.data_as(C.c_void_p), a.nbytes))
    lcu.check(lcu.lib.lcu_memset(kc.ptr, 0, kc.nbytes))
    lcu.check(lcu.lib.lcu_memset(vc.ptr, 0, vc.nbytes))
    lcu.check(fn(dq.ptr, dk.ptr, dv.ptr, kc.ptr, vc.ptr, pos0, m, dim, n_heads, ctx, None))
    lcu.check(lcu.lib.lcu_synchronize())
    return dq.to_host(np.uint16, (m, dim)), kc.to_host(np.uint16, (ctx * dim,)), vc.to_host(np.uint16, (ctx * dim,))


def free_bytes(lcu):
    free, total = C.c_uint64(0), C.c_uint64(0)
    lcu.check(lcu.lib.lcu_mem_info(C.byref(free), C.byref(total)))
    return free.value


def test_static_variant_equals_allocating_variant_twice_in_a_row(lcu):
    rng = np.random.default_rng(42)
    # second call: other head_dim and positions, so the table left by the first call is stale everywhere it is reused
    for m, dim, n_heads, pos0, ctx in ((5, 256, 2, 9, 64), (3, 256, 4, 40, 48)):
        q, k, v = (rng.standard_normal((m, dim)).astype(np.float16).view(np.uint16) for _ in range(3))
        want = run(lcu, lcu.lib.lcu_rope_scatter, q, k, v, n_heads, pos0, ctx)
        got = run(lcu, lcu.lib.lcu_rope_scatter_static, q, k, v, n_heads, pos0, ctx)
        for a, b in zip(got, want):
            assert (a == b).all()  # same kernels, same table values: bit identical
        # and directly against the CPU restatement of the reference's rotary kernel (llama_cu.cu:368-389)
        qo, ko = np.zeros_like(q), np.zeros_like(k)
        O.lib().orc_rotary(qo.reshape(-1), q.reshape(-1), m, dim, n_heads, pos0, 10000.0)
        O.lib().orc_rotary(ko.reshape(-1), k.reshape(-1), m, dim, n_heads, pos0, 10000.0)
        hd = dim // n_heads
        k_rows = got[1].reshape(n_heads, ctx, hd)[:, pos0:pos0 + m, :].transpose(1, 0, 2).reshape(m, dim)
        v_rows = got[2].reshape(n_heads, ctx, hd)[:, pos0:pos0 + m, :].transpose(1, 0, 2).reshape(m, dim)
        assert np.abs(f32(got[0]) - f32(qo)).max() <= 4e-3 and np.abs(f32(k_rows) - f32(ko)).max() <= 4e-3  # powf/sinf/cosf: device vs libm
        assert (v_rows == v).all()


def test_static_variant_takes_no_device_memory_after_its_first_call(lcu):
    rng = np.random.default_rng(43)
    m, dim, n_heads, pos0, ctx = 4, 256, 2, 3, 32
    q, k, v = (rng.standard_normal((m, dim)).astype(np.float16).view(np.uint16) for _ in range(3))
    bufs = [lcu.DeviceBuffer(q.nbytes), lcu.DeviceBuffer(k.nbytes), lcu.DeviceBuffer(v.nbytes), lcu.DeviceBuffer(ctx * dim * 2),
            lcu.DeviceBuffer(ctx * dim * 2)]
    run(lcu, lcu.lib.lcu_rope_scatter_static, q, k, v, n_heads, pos0, ctx, bufs)  # start-up call: module load, address look-up
    before = free_bytes(lcu)
    for pos in (3, 7, 20):
        run(lcu, lcu.lib.lcu_rope_scatter_static, q, k, v, n_heads, pos, ctx, bufs)
        assert free_bytes(lcu) == before


def test_static_variant_rejects_requests_beyond_its_table(lcu):
    d = lcu.DeviceBuffer(1 << 12)
    rc = lcu.lib.lcu_rope_scatter_static(d.ptr, d.ptr, d.ptr, d.ptr, d.ptr, 4096, 1, 256, 2, 8192, None)
    assert rc == 2 and b"exceed the static table" in lcu.lib.lcu_last_error()
