"""The sampler the reference has commented out (llama_cu.cu:1202-1203: std::discrete_distribution over the fp16
probabilities) as a device kernel, and the context roll-over that keeps the cache instead of feeding the prompt again
(the reference's client re-prompts: main.cpp:83-87)."""
import ctypes as C

import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu
L = O.lib()
SMALL = dict(dim=256, n_heads=2, n_layers=3, n_vocab=1000)


def f16(a):
    return np.asarray(a, np.float32).astype(np.float16).view(np.uint16)


def f32(u):
    return np.asarray(u, np.uint16).view(np.float16).astype(np.float32)


def sample(lcu, probs_u16, u):
    d = lcu.DeviceBuffer.from_host(probs_u16)
    tok = C.c_int(-1)
    lcu.check(lcu.lib.lcu_sample_token(d.ptr, probs_u16.size, u, C.byref(tok), None))
    return tok.value


def test_sample_token_equals_the_host_restatement(lcu):
    rng = np.random.default_rng(1)
    for n in (1000, 32000, 7):
        logits = rng.standard_normal(n) * 3
        p = np.exp(logits - logits.max())
        probs = f16(p / p.sum())
        probs[rng.integers(0, n, n // 10)] = 0  # holes: a zero-probability token is never returned
        for u in [0.0, 1e-7, 0.25, 0.5, 0.75, 0.999999, float(np.float32(1) - np.float32(2.0 ** -24))] + list(rng.random(20)):
            t = sample(lcu, probs, float(np.float32(u)))
            assert t == L.orc_sample_token(probs, n, float(np.float32(u))), (n, u)
            assert f32(probs)[t] > 0
    one_hot = np.zeros(500, np.uint16)
    one_hot[123] = f16(1.0)
    assert all(sample(lcu, one_hot, u) == 123 for u in (0.0, 0.5, 0.99))
    with pytest.raises(lcu.LcuError, match="outside"):
        sample(lcu, one_hot, 1.0)


def test_sample_token_follows_the_distribution(lcu):
    probs = f16(np.array([0.5, 0.25, 0.125, 0.0625, 0.0625]))
    d = lcu.DeviceBuffer.from_host(probs)
    tok = C.c_int(0)
    counts = np.zeros(5)
    n = 4000
    for i in range(n):
        lcu.check(lcu.lib.lcu_sample_token(d.ptr, 5, lcu.lib.lcu_sampler_uniform(99, i), C.byref(tok), None))
        counts[tok.value] += 1
    expected = f32(probs) * n
    assert (np.abs(counts - expected) < 5 * np.sqrt(expected)).all(), counts
    # the host and device generators are one recipe
    for i in (0, 1, 77, 1 << 20):
        assert lcu.lib.lcu_sampler_uniform(1234, i) == L.orc_sampler_uniform(1234, i)


def test_context_sampling_is_seeded_and_matches_the_restatement(lcu):
    model = lcu.Model.synthetic(block_size=0, seed=7, scale=0.08, **SMALL)
    prompt = O.synth_tokens(9, 7, lo=3, hi=1000)
    runs = []
    for seed in (5, 5, 6):
        ctx = lcu.Context(model, context_len=64, temperature=0.8)
        greedy_first = ctx.next_token(prompt)
        ctx.clear_tokens()
        ctx.set_sampling(1, seed)
        assert ctx.kernels_per_step() == 1 + 5 * 3 + 3
        toks = [ctx.next_token(prompt)]
        for step in range(12):
            probs = ctx.probs()
            # the token just returned was drawn from the probabilities of the step that produced it
            u = lcu.lib.lcu_sampler_uniform(seed, 9 + step)
            assert toks[-1] == L.orc_sample_token(probs, 1000, u), step
            toks.append(ctx.next_token([toks[-1]]))
        chained, _ = ctx.decode_chained(toks[-1], 8)  # the captured step samples too, and logs the sampled tokens
        ctx.set_sampling(0, 0)
        assert ctx.kernels_per_step() == 1 + 5 * 3 + 2
        runs.append((toks, list(chained), greedy_first))
        ctx.close()
    assert runs[0][:2] == runs[1][:2]          # same seed: the same run
    assert runs[0][0] != runs[2][0]            # another seed: another run
    assert runs[0][0][1:] != [runs[0][2]] * 12
    model.close()


def test_rollover_operator_against_the_rotary_restatement(lcu):
    """Rows [first, first + keep) of a layer's caches move to [0, keep): values bit for bit, keys as if they had been
    rotated at their new positions (one more rounding to half than a fresh rotation: 2 ulp of tolerance on top of the
    device-vs-libm difference)."""
    rng = np.random.default_rng(3)
    for H, hd, T, first in ((2, 128, 40, 24), (3, 64, 50, 7), (1, 128, 33, 32)):
        keep = T - first
        dim = H * hd
        k, v = f16(rng.standard_normal((T, dim))), f16(rng.standard_normal((T, dim)))
        q = f16(rng.standard_normal((T, dim)))
        _, kc, vc = lcu.rope_scatter(q, k, v, H, 0, T)  # caches as a context holds them: keys rotated at 0 .. T-1
        dk, dv = lcu.DeviceBuffer.from_host(kc), lcu.DeviceBuffer.from_host(vc)
        lcu.check(lcu.lib.lcu_rollover(dk.ptr, dv.ptr, H, T, hd, first, keep, None))
        lcu.check(lcu.lib.lcu_synchronize())
        kc2, vc2 = dk.to_host(np.uint16, (H, T, hd)), dv.to_host(np.uint16, (H, T, hd))
        want = np.zeros((keep, dim), np.uint16)
        L.orc_rotary(want.reshape(-1), np.ascontiguousarray(k[first:]).reshape(-1), keep, dim, H, 0, 10000.0)
        got = kc2[:, :keep].transpose(1, 0, 2).reshape(keep, dim)
        assert np.abs(f32(got) - f32(want)).max() <= 8e-3 * max(1.0, float(np.abs(f32(want)).max())), (H, hd, first)
        assert (vc2[:, :keep] == vc[:, first:T]).all()
        assert (kc2[:, keep:] == kc[:, keep:]).all() or first < keep  # rows past `keep` are only touched as sources


def test_context_rollover_continues_past_the_old_limit(lcu):
    model = lcu.Model.synthetic(block_size=0, seed=11, scale=0.08, **SMALL)
    ctx = lcu.Context(model, context_len=48, temperature=0.8)
    prompt = O.synth_tokens(40, 11, lo=3, hi=1000)
    t = ctx.next_token(prompt)
    assert ctx.tokens_left() == 8
    ctx.rollover(16)
    assert ctx.tokens_left() == 32
    for _ in range(20):  # more steps than were left before the roll-over
        t = ctx.next_token([t])
        p = f32(ctx.probs())
        assert np.isfinite(p).all() and abs(float(p.sum()) - 1.0) < 2e-2 and 0 <= t < 1000
    with pytest.raises(lcu.LcuError, match="rollover"):
        ctx.rollover(100)
    ctx.close()
    model.close()
