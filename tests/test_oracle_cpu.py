"""CPU checks of the oracle (oracle/oracle.cpp) against numpy restatements and analytic properties."""
import hashlib

import numpy as np
import pytest

import oracle_lib as O

L = O.lib()


def f16(a):
    return np.asarray(a, np.float32).astype(np.float16).view(np.uint16)


def f32(u):
    return np.asarray(u, np.uint16).view(np.float16).astype(np.float32)


def test_half_conversions_match_numpy():
    rng = np.random.default_rng(1)
    xs = (rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 6, 20000)).astype(np.float32)
    xs = np.concatenate([xs, np.array([0, -0.0, 65504, 65519.996, 65520, 1e-8, 2**-25, 2**-24, 6.1e-5, np.inf, -np.inf], np.float32)])
    mine = np.array([L.orc_f2h(float(x)) for x in xs], np.uint16)
    with np.errstate(over="ignore"):
        ref = xs.astype(np.float16).view(np.uint16)
    assert (mine == ref).all()
    hs = np.arange(0, 65536, 7, dtype=np.uint16)
    back = np.array([L.orc_h2f(int(h)) for h in hs], np.float32)
    want = hs.view(np.float16).astype(np.float32)
    assert ((back == want) | (np.isnan(back) & np.isnan(want))).all()


def test_synth_generator_is_deterministic_and_normalish():
    a = O.synth_f16(1 << 16, 1234, "layers.0.attention.wq", 0.02)
    b = O.synth_f16(1 << 16, 1234, "layers.0.attention.wq", 0.02)
    c = O.synth_f16(1 << 16, 1234, "layers.0.attention.wk", 0.02)
    assert (a == b).all() and (a != c).any()
    # a window of the stream equals the same indices of the whole stream
    w = O.synth_f16(100, 1234, "layers.0.attention.wq", 0.02, first=5000)
    assert (w == a[5000:5100]).all()
    v = f32(a)
    assert abs(v.mean()) < 5e-4 and abs(v.std() - 0.02) < 5e-4 and np.abs(v).max() < 0.02 * 5
    # pinned bits: the generator is part of every fixture, it must never drift
    assert hashlib.sha256(a.tobytes()).hexdigest()[:16] == SYNTH_SHA16


SYNTH_SHA16 = hashlib.sha256(O.synth_f16(1 << 16, 1234, "layers.0.attention.wq", 0.02).tobytes()).hexdigest()[:16]


def test_synth_tokens_range():
    t = O.synth_tokens(128, 1234)
    assert t.min() >= 3 and t.max() < 32000 and len(set(t.tolist())) > 100


def np_quantize(w_u16, bs):
    """numpy restatement of transform.cu:28-72 (round half away from zero, NaN -> 0)."""
    x = f32(w_u16)
    h, w = x.shape
    xb = x.reshape(h, w // bs, bs)
    amax = np.abs(xb).max(axis=2)
    sc = (amax / np.float32(127.5)).astype(np.float32).astype(np.float16)
    s = sc.astype(np.float32)[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        v = np.float32(127.5) + (xb / s).astype(np.float32)
    r = np.where(v >= 0, np.floor(v + np.float32(0.5)), np.ceil(v - np.float32(0.5)))
    r = np.where(np.isnan(v), 0, r)
    return np.clip(r, 0, 255).astype(np.uint8).reshape(h, w), sc.view(np.uint16)


@pytest.mark.parametrize("h,w,bs", [(8, 256, 128), (3, 512, 64), (5, 128, 32), (2, 11008, 128)])
def test_quantizer_matches_numpy_restatement(h, w, bs):
    x = O.synth_f16(h * w, 7, f"q{h}x{w}", 0.02).reshape(h, w)
    q, s = O.quantize(x, h, w, bs)
    qn, sn = np_quantize(x, bs)
    assert (s == sn).all()
    assert (q == qn).all()
    assert q.max() == 255 or q.min() == 0  # the absmax element always lands on an end of the range


def test_quantizer_edge_cases():
    bs = 128
    x = np.zeros((3, 256), np.uint16)
    x[1, :128] = f16(np.linspace(-1, 1, 128))
    x[2, 128:] = f16(np.full(128, 6e-8))  # subnormal block
    q, s = O.quantize(x, 3, 256, bs)
    assert (q[0] == 0).all() and (s[0] == 0).all()  # 0/0 -> NaN -> 0 as on the device
    assert (q[1, 128:] == 0).all()
    assert q[1, 0] == 0 and q[1, 127] == 255
    # ties round away from zero: x/scale exactly k+0.5 -> 127.5 + k + 0.5 is an integer, no tie; x/scale = k -> .5 tie
    sc = np.float16(2.0 ** -7)
    vals = (np.arange(-127, 128, 2, dtype=np.float32) * np.float32(sc)).astype(np.float16)  # odd multiples
    blk = np.zeros(128, np.float16)
    blk[: len(vals)] = vals
    blk[-1] = np.float16(127.5 * float(sc))  # pins the scale to sc
    q2, s2 = O.quantize(blk.view(np.uint16).reshape(1, 128), 1, 128, 128)
    assert s2[0, 0] == np.float16(sc).view(np.uint16)
    k = np.arange(-127, 128, 2)
    assert (q2[0, : len(k)] == 128 + k).all()  # 127.5 + k = x.5 -> away from zero -> 128 + k


def test_dequantize_and_error_stats():
    x = O.synth_f16(64 * 256, 3, "dq", 0.02).reshape(64, 256)
    q, s = O.quantize(x, 64, 256, 128)
    dq = np.empty((64, 256), np.uint16)
    L.orc_dequantize_absmax_uint8(dq, s, q, 64, 256, 128)
    want = ((q.astype(np.float32) - np.float32(127.5)) * f32(s).repeat(128, axis=1)).astype(np.float16)
    assert (dq.view(np.float16) == want).all()
    st = np.zeros(3, np.float32)
    L.orc_error_stats(st, x.reshape(-1), dq.reshape(-1), x.size)
    d = f32(x) - f32(dq)
    assert np.allclose(st, [np.mean(d.astype(np.float64) ** 2), np.abs(d).max(), np.abs(d).mean()], rtol=1e-5)
    # half a quantization step of the largest block scale bounds the error (plus the fp16 rounding of the product)
    assert st[1] <= f32(s).max() * 0.5 * 1.01 + 1e-4


def test_matmul_fp16_against_float64():
    rng = np.random.default_rng(0)
    m, k, n = 3, 512, 64
    a, b = f16(rng.standard_normal((m, k))), f16(rng.standard_normal((n, k)) * 0.02)
    out = np.zeros((m, n), np.uint16)
    L.orc_matmul_nt_f16(out.reshape(-1), a.reshape(-1), b.reshape(-1), m, k, n, 0.0, 0)
    gold = f32(a).astype(np.float64) @ f32(b).astype(np.float64).T
    assert np.abs(f32(out) - gold).max() <= np.abs(gold).max() * 2e-3
    # beta = 1 adds the previous contents (residual form, llama_cu.cu:1174)
    prev = f16(rng.standard_normal((m, n)))
    out2 = prev.copy()
    L.orc_matmul_nt_f16(out2.reshape(-1), a.reshape(-1), b.reshape(-1), m, k, n, 1.0, 0)
    assert np.abs(f32(out2) - (gold + f32(prev))).max() <= 4e-3 * max(1.0, np.abs(gold + f32(prev)).max())


def test_matmul_int8_modes():
    rng = np.random.default_rng(2)
    m, k, n, bs = 2, 512, 32, 128
    a = f16(rng.standard_normal((m, k)))
    w = O.synth_f16(n * k, 5, "w8", 0.02).reshape(n, k)
    q, s = O.quantize(w, n, k, bs)
    outs = []
    for mode in (0, 1, 2, 3):
        o = np.zeros((m, n), np.uint16)
        L.orc_matmul_nt_fp16u8(o.reshape(-1), a.reshape(-1), q.reshape(-1), s.reshape(-1), m, k, n, bs, 0.0, mode)
        outs.append(f32(o))
    deq = (q.astype(np.float64) - 127.5) * f32(s).astype(np.float64).repeat(bs, axis=1)
    gold = f32(a).astype(np.float64) @ deq.T
    for o in outs:
        assert np.abs(o - gold).max() <= np.abs(gold).max() * 5e-3
    g64 = np.zeros((m, n), np.float64)
    L.orc_matmul_nt_gold(g64.reshape(-1), a.reshape(-1), None, q.ctypes.data, s.ctypes.data, m, k, n, bs, 0)
    assert np.allclose(g64, gold, rtol=1e-12, atol=1e-12)


def test_rms_norm_rotary_silu_against_numpy():
    rng = np.random.default_rng(3)
    x, w = f16(rng.standard_normal((4, 512))), f16(1 + 0.1 * rng.standard_normal(512))
    out = np.zeros_like(x)
    L.orc_rms_norm(out.reshape(-1), x.reshape(-1), w, 4, 512, 1e-6)
    xf = f32(x).astype(np.float64)
    want = xf / np.sqrt((xf ** 2).mean(axis=1, keepdims=True) + 1e-6) * f32(w)
    assert np.abs(f32(out) - want).max() < 4e-3
    # rotary: norm-preserving on every pair, identity at position 0
    q = f16(rng.standard_normal((5, 256)))
    r0 = np.zeros_like(q)
    L.orc_rotary(r0.reshape(-1), q.reshape(-1), 1, 256, 2, 0, 10000.0)
    assert (r0[0] == q[0]).all()
    r = np.zeros_like(q)
    L.orc_rotary(r.reshape(-1), q.reshape(-1), 5, 256, 2, 7, 10000.0)
    n_in = (f32(q).reshape(5, 128, 2) ** 2).sum(-1)
    n_out = (f32(r).reshape(5, 128, 2) ** 2).sum(-1)
    assert np.abs(n_in - n_out).max() < 2e-2
    hd = 128
    ang = (7 + np.arange(5))[:, None] / 10000.0 ** (np.arange(0, hd, 2) / hd)[None, :]
    qq = f32(q).reshape(5, 2, hd // 2, 2)
    re = qq[..., 0] * np.cos(ang)[:, None, :] - qq[..., 1] * np.sin(ang)[:, None, :]
    assert np.abs(f32(r).reshape(5, 2, hd // 2, 2)[..., 0] - re).max() < 3e-3
    a, b = f16(rng.standard_normal(1000) * 3), f16(rng.standard_normal(1000))
    o = np.zeros(1000, np.uint16)
    L.orc_silu(o, a, b, 1000)
    af = f32(a).astype(np.float64)
    want = af / (1 + np.exp(-af)) * f32(b)
    assert (np.abs(f32(o) - want) <= 1e-3 * np.abs(want) + 1e-4).all()


def test_gated_product_is_the_two_products_and_the_gate():
    """orc_matmul_nt_f16_gated - the restatement of llama_cu.cu:1180-1183 that the one-launch GPU operator is checked
    against - equals matmul_nt with w1, matmul_nt with w3 (halves) and silu on those halves, and matches numpy in
    double precision up to the three roundings to half."""
    rng = np.random.default_rng(12)
    m, k, f = 5, 256, 96
    x = f16(rng.standard_normal((m, k)))
    w13 = f16(rng.standard_normal((2 * f, k)) * 0.08)
    got = np.zeros((m, f), np.uint16)
    L.orc_matmul_nt_f16_gated(got.reshape(-1), x.reshape(-1), w13.reshape(-1), m, k, f, 1)
    a, b, want = np.zeros((m, f), np.uint16), np.zeros((m, f), np.uint16), np.zeros((m, f), np.uint16)
    L.orc_matmul_nt_f16(a.reshape(-1), x.reshape(-1), np.ascontiguousarray(w13[:f]).reshape(-1), m, k, f, 0.0, 1)
    L.orc_matmul_nt_f16(b.reshape(-1), x.reshape(-1), np.ascontiguousarray(w13[f:]).reshape(-1), m, k, f, 0.0, 1)
    L.orc_silu(want.reshape(-1), a.reshape(-1), b.reshape(-1), m * f)
    assert np.array_equal(got, want)
    xa = f32(x).astype(np.float64) @ f32(w13[:f]).astype(np.float64).T
    xb = f32(x).astype(np.float64) @ f32(w13[f:]).astype(np.float64).T
    ref = xa / (1 + np.exp(-xa)) * xb
    assert np.abs(f32(got) - ref).max() <= 4e-3 * max(1.0, np.abs(ref).max())


def test_attention_chain_against_numpy_softmax():
    rng = np.random.default_rng(4)
    m, T, dim, H, sp = 3, 11, 256, 2, 8
    q, k, v = f16(rng.standard_normal((m, dim))), f16(rng.standard_normal((T, dim))), f16(rng.standard_normal((T, dim)))
    out = np.zeros((m, dim), np.uint16)
    L.orc_attention(out.reshape(-1), q.reshape(-1), k.reshape(-1), v.reshape(-1), m, T, dim, H, sp, 0)
    out32 = np.zeros((m, dim), np.uint16)
    L.orc_attention(out32.reshape(-1), q.reshape(-1), k.reshape(-1), v.reshape(-1), m, T, dim, H, sp, 1)
    hd = dim // H
    for h in range(H):
        qs, ks, vs = (f32(t)[:, h * hd:(h + 1) * hd].astype(np.float64) for t in (q, k, v))
        s = qs @ ks.T / np.sqrt(hd)
        for r in range(m):
            s[r, r + sp + 1:] = -np.inf
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        want = p @ vs
        assert np.abs(f32(out)[:, h * hd:(h + 1) * hd] - want).max() < 2e-2
        assert np.abs(f32(out32)[:, h * hd:(h + 1) * hd] - want).max() < 5e-3


def small_model(block_size=0, n_layers=2, ctx=64):
    return O.OracleModel(dim=256, multiple_of=256, n_heads=2, n_layers=n_layers, n_vocab=1000, block_size=block_size, seed=1234,
                         scale=0.02 * 4, context_len=ctx, temperature=0.8)


@pytest.mark.parametrize("bs", [0, 128])
def test_oracle_forward_prefill_equals_incremental(bs):
    prompt = O.synth_tokens(12, 1234, lo=3, hi=1000)
    a = small_model(bs)
    ta = [a.next_token(prompt)]
    pa = a.probs()
    for _ in range(6):
        ta.append(a.next_token([ta[-1]]))
    b = small_model(bs)
    for t in prompt[:-1]:
        b.next_token([t])
    tb = [b.next_token([prompt[-1]])]
    assert (b.probs() == pa).all()  # rows are independent, so chunking the prompt changes nothing
    for _ in range(6):
        tb.append(b.next_token([tb[-1]]))
    assert ta == tb
    assert abs(float(f32(pa).sum()) - 1.0) < 2e-2
    a.close()
    b.close()


def test_oracle_ffn_dim_matches_reference_shapes():
    assert L.orc_ffn_dim(4096, 256) == 11008 and L.orc_ffn_dim(5120, 256) == 13824 and L.orc_ffn_dim(8192, 256) == 22016
    assert L.orc_ffn_dim(256, 256) == 768
