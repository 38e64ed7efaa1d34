"""End-to-end parity of the forward pass: new library vs the CPU oracle (small shapes) and vs the
reference's own llama_context::next_token (when the reference library is present)."""
import os

import numpy as np
import pytest

import oracle_lib as O
import ref_lib as R

pytestmark = pytest.mark.gpu

SMALL = dict(dim=256, n_heads=2, n_layers=3, n_vocab=1000)


def f32(u):
    return np.asarray(u, np.uint16).view(np.float16).astype(np.float32)


def run_tokens(ctx, prompt, steps):
    toks = [ctx.next_token(prompt)]
    for _ in range(steps):
        toks.append(ctx.next_token([toks[-1]]))
    return toks


@pytest.fixture
def u8_mode(lcu, request):
    """int8_factored for the duration of a test: 1 = scale factored out per block (default), 0 = every weight rounded to
    half before the product, as the reference's tensor-core kernel does (llama_cu.cu:287-289)."""
    lcu.check(lcu.lib.lcu_set_tuning(b"int8_factored", request.param))
    yield request.param
    lcu.check(lcu.lib.lcu_set_tuning(b"int8_factored", 1))


@pytest.mark.parametrize("bs,prompt_len,u8_mode", [(0, 12, 1), (128, 12, 1), (0, 40, 1), (128, 40, 1), (128, 12, 0), (128, 40, 0), (64, 12, 0),
                                                   (64, 12, 1), (32, 12, 1)], indirect=["u8_mode"])
def test_small_model_matches_oracle(lcu, bs, prompt_len, u8_mode):
    """12-token prompts go through the multi-row GEMV passes; 40-token prompts through the tcgen05 GEMM (u8 weights
    expanded to fp16 first) and the tiled prompt attention.  u8 models run in both weight modes of the decode GEMV and
    with every supported block size."""
    scale = 0.08
    model = lcu.Model.synthetic(block_size=bs, seed=1234, scale=scale, **SMALL)
    ctx = lcu.Context(model, context_len=64, temperature=0.8)
    om = O.OracleModel(dim=256, multiple_of=256, n_heads=2, n_layers=3, n_vocab=1000, block_size=bs, seed=1234, scale=scale,
                       context_len=64, temperature=0.8)
    # identical weights on both sides (generator and quantizer are bit exact)
    wq = model.tensor_host("layers.1.attention.wq", 0, np.uint8 if bs else np.uint16)
    want = O.synth_f16(256 * 256, 1234, "layers.1.attention.wq", scale)
    if bs:
        q, s = O.quantize(want.reshape(256, 256), 256, 256, bs)
        assert (wq == q.reshape(-1)).all() and (model.tensor_host("layers.1.attention.wq", 1) == s.reshape(-1)).all()
    else:
        assert (wq == want).all()
    prompt = O.synth_tokens(prompt_len, 1234, lo=3, hi=1000)
    mine, theirs = [], []
    # u8 weights: once through the GEMV passes (threshold raised), once through dequantization + tcgen05 GEMM (default)
    lcu.check(lcu.lib.lcu_set_tuning(b"prefill_u8_deq_min_rows", 2 if prompt_len >= 40 else 1000))
    try:
        t = ctx.next_token(prompt)
    finally:
        lcu.check(lcu.lib.lcu_set_tuning(b"prefill_u8_deq_min_rows", 2))
    to = om.next_token(prompt)
    for step in range(20):
        p, po = f32(ctx.probs()), f32(om.probs())
        assert np.abs(p - po).max() <= 0.02 * po.max() + 1e-4, step  # same distribution up to summation order / libm ulps
        h, ho = f32(ctx.hidden()), f32(om.last_hidden())
        assert np.abs(h - ho).max() <= 0.02 * np.abs(ho).max(), step
        mine.append(t)
        theirs.append(to)
        # teacher forcing on the oracle's token keeps the two runs on the same trajectory
        t, to = ctx.next_token([to]), om.next_token([to])
    agree = np.mean(np.array(mine) == np.array(theirs))
    assert agree >= 0.9, (mine, theirs)
    assert ctx.tokens_left() == 64 - prompt_len - 20
    om.close()
    ctx.close()
    model.close()


def test_long_prompt_attention_paths_against_oracle(lcu):
    """A 300-token prompt through the one-kernel tcgen05 attention (2), the three-kernel tcgen05 path with its score buffer
    (1) and the fused warp-level kernel (0): all must reproduce the oracle's next-token distribution, and a decode step after either must too
    (the KV cache they leave behind is the same)."""
    scale = 0.08
    cfg = dict(dim=256, multiple_of=256, n_heads=2, n_layers=3, n_vocab=1000)
    model = lcu.Model.synthetic(block_size=0, seed=99, scale=scale, **cfg)
    om = O.OracleModel(block_size=0, seed=99, scale=scale, context_len=320, temperature=0.8, **cfg)
    prompt = O.synth_tokens(300, 99, lo=3, hi=1000)
    to = om.next_token(prompt)
    po = f32(om.probs())
    to2 = om.next_token([to])
    po2 = f32(om.probs())
    try:
        for tc in (2, 1, 0):
            lcu.check(lcu.lib.lcu_set_tuning(b"prefill_attn_tc", tc))
            lcu.check(lcu.lib.lcu_set_tuning(b"prefill_attn_tc_min_rows", 2))
            ctx = lcu.Context(model, context_len=320, temperature=0.8)
            t = ctx.next_token(prompt)
            pr = f32(ctx.probs())
            assert np.abs(pr - po).max() <= 0.02 * po.max() + 1e-4, tc
            ctx.next_token([to])
            pr2 = f32(ctx.probs())
            assert np.abs(pr2 - po2).max() <= 0.02 * po2.max() + 1e-4, tc
            ctx.close()
    finally:
        lcu.check(lcu.lib.lcu_set_tuning(b"prefill_attn_tc", 2))
        lcu.check(lcu.lib.lcu_set_tuning(b"prefill_attn_tc_min_rows", 384))
    om.close()
    model.close()


@pytest.mark.parametrize("bs", [0, 128])
def test_long_prompt_with_gate_in_the_gemm_epilogue_against_oracle(lcu, bs):
    """A 300-token prompt with w1|w3 and the SiLU gate as one launch (both tile widths) and as product + gate kernel
    (llama_cu.cu:1180-1183): each reproduces the oracle's next-token distribution, and the one-launch passes give the
    same token as the two-step pass."""
    scale = 0.08
    cfg = dict(dim=256, multiple_of=256, n_heads=2, n_layers=3, n_vocab=1000)
    model = lcu.Model.synthetic(block_size=bs, seed=77, scale=scale, **cfg)
    om = O.OracleModel(block_size=bs, seed=77, scale=scale, context_len=320, temperature=0.8, **cfg)
    prompt = O.synth_tokens(300, 77, lo=3, hi=1000)
    om.next_token(prompt)
    po = f32(om.probs())
    tokens = []
    try:
        for mode in (0, 256, 512, -1):
            lcu.check(lcu.lib.lcu_set_tuning(b"prefill_gate_fused", mode))
            ctx = lcu.Context(model, context_len=320, temperature=0.8)
            tokens.append(ctx.next_token(prompt))
            pr = f32(ctx.probs())
            assert np.abs(pr - po).max() <= 0.02 * po.max() + 1e-4, mode
            ctx.close()
    finally:
        lcu.check(lcu.lib.lcu_set_tuning(b"prefill_gate_fused", -1))
    assert len(set(tokens)) == 1, tokens
    om.close()
    model.close()


def test_u8_prompt_from_the_fp16_shadow_equals_the_per_pass_expansion(lcu):
    """u8 models: a prompt of 9 tokens or more reads fp16 copies of the layer matrices - expanded once into a shadow of
    the model where the GPU has room, or into scratch on every pass.  Same kernel, same halves (llama_cu.cu:287-289):
    the two must give the same probabilities bit for bit.  The shadow follows the weights: after a tensor was handed
    out and rewritten, the next prompt sees the new values."""
    cfg = dict(dim=256, multiple_of=256, n_heads=2, n_layers=3, n_vocab=1000)
    prompt = O.synth_tokens(40, 31, lo=3, hi=1000)
    out = {}
    try:
        for mode in (0, 1):
            lcu.check(lcu.lib.lcu_set_tuning(b"prefill_u8_shadow", mode))
            model = lcu.Model.synthetic(block_size=128, seed=31, scale=0.08, **cfg)
            ctx = lcu.Context(model, context_len=64, temperature=0.8)
            tok = ctx.next_token(prompt)
            assert (model.shadow_bytes() > 0) == (mode == 1)
            probs = np.asarray(ctx.probs(), np.uint16).copy()
            # rewrite one matrix (all bytes 200) and run the prompt again
            ptr, nbytes, _ = model.tensor("layers.1.feed_forward.w2")
            lcu.check(lcu.lib.lcu_memcpy_h2d(ptr, lcu._ptr(np.full(nbytes, 200, np.uint8)), nbytes))
            ctx.clear_tokens()
            tok2 = ctx.next_token(prompt)
            probs2 = np.asarray(ctx.probs(), np.uint16).copy()
            out[mode] = (tok, probs, tok2, probs2)
            ctx.close()
            model.close()
    finally:
        lcu.check(lcu.lib.lcu_set_tuning(b"prefill_u8_shadow", 1))
    assert out[0][0] == out[1][0] and np.array_equal(out[0][1], out[1][1])
    assert out[0][2] == out[1][2] and np.array_equal(out[0][3], out[1][3])
    assert not np.array_equal(out[1][1], out[1][3])  # the rewritten matrix did change the result


def test_fresh_contexts_repeat_the_same_distribution(lcu):
    """A context is usable the moment it is created: its zeroed arenas and its RoPE table are ordered on the context's
    own stream.  Twenty contexts in a row, each used at once with a context length whose arenas take a while to clear,
    must all produce the same probabilities and the same next token."""
    model = lcu.Model.synthetic(block_size=0, seed=5, scale=0.08, **SMALL)
    prompt = O.synth_tokens(24, 5, lo=3, hi=1000)
    first = None
    for _ in range(20):
        ctx = lcu.Context(model, context_len=4096, temperature=0.8)
        tok = ctx.next_token(prompt)
        got = (tok, np.asarray(ctx.probs(), np.uint16).copy(), ctx.next_token([tok]))
        ctx.close()
        if first is None:
            first = got
        assert got[0] == first[0] and got[2] == first[2]
        assert np.array_equal(got[1], first[1])
    model.close()


def test_chained_decode_equals_host_loop_and_graph_equals_direct(lcu):
    model = lcu.Model.synthetic(block_size=0, seed=7, scale=0.08, **SMALL)
    prompt = O.synth_tokens(9, 7, lo=3, hi=1000)
    runs = {}
    for name, graph, pdl in (("graph+pdl", 1, 1), ("direct", 0, 0), ("graph", 1, 0), ("pdl", 0, 1)):
        lcu.check(lcu.lib.lcu_set_tuning(b"use_graph", graph))
        lcu.check(lcu.lib.lcu_set_tuning(b"use_pdl", pdl))
        ctx = lcu.Context(model, context_len=64, temperature=0.8)
        first = ctx.next_token(prompt)
        host = [first]
        for _ in range(16):
            host.append(ctx.next_token([host[-1]]))
        ctx.clear_tokens()
        assert ctx.next_token(prompt) == first
        chained, ms = ctx.decode_chained(first, 16)
        assert chained.tolist() == host[1:], name
        assert ms > 0 and ctx.tokens_left() == 64 - 9 - 16
        runs[name] = host
        ctx.close()
    lcu.check(lcu.lib.lcu_set_tuning(b"use_graph", 1))
    lcu.check(lcu.lib.lcu_set_tuning(b"use_pdl", 1))
    assert all(r == runs["direct"] for r in runs.values())  # every launch mode is bit-deterministic and identical
    model.close()


def test_context_limits_and_errors(lcu):
    model = lcu.Model.synthetic(block_size=0, seed=7, scale=0.08, **SMALL)
    ctx = lcu.Context(model, context_len=16, temperature=0.8)
    with pytest.raises(lcu.LcuError, match="exceed the context length"):
        ctx.next_token(list(range(3, 20)))
    with pytest.raises(lcu.LcuError, match="outside the vocabulary"):
        ctx.next_token([5000])
    ctx.next_token(list(range(3, 19)))  # exactly fills the context
    assert ctx.tokens_left() == 0
    with pytest.raises(lcu.LcuError):
        ctx.next_token([3])
    ctx.clear_tokens()
    assert ctx.tokens_left() == 16 and ctx.memory_usage() > 0
    ctx.close()
    model.close()
    with pytest.raises(lcu.LcuError, match="multiple of 256"):
        lcu.Model.synthetic(dim=200, n_heads=2, n_layers=1, n_vocab=1000)


@pytest.mark.parametrize("bs", [0, 128])
def test_weight_directory_round_trip(lcu, tmp_path, bs):
    """The on-disk layout is the reference's: a saved model loads back bit-identically, the CPU oracle
    reads the same files, and (when present) the reference's own loader runs them."""
    model = lcu.Model.synthetic(block_size=bs, seed=11, scale=0.08, **SMALL)
    d = str(tmp_path / "m")
    model.save(d)
    names = sorted(os.listdir(d))
    assert "params" in names and "tok_embeddings.weight__1000_256" in names and "layers.2.feed_forward.w2.weight__256_768" in names
    assert ("layers.0.attention.wq.scale__256_2" in names) == bool(bs)
    assert os.path.getsize(os.path.join(d, "params")) == 40
    again = lcu.Model.load(d)
    for name in ("tok_embeddings", "layers.2.feed_forward.w3", "norm"):
        assert (again.tensor_host(name, 0, np.uint8) == model.tensor_host(name, 0, np.uint8)).all()
    # the reference's way of loading (file mapping + one pageable copy per tensor) is kept as the loader's baseline
    lcu.check(lcu.lib.lcu_set_tuning(b"loader_staged", 0))
    try:
        mapped = lcu.Model.load(d)
    finally:
        lcu.check(lcu.lib.lcu_set_tuning(b"loader_staged", 1))
    for name in ("tok_embeddings", "output", "layers.0.attention.wq", "layers.2.feed_forward.w3", "norm"):
        for which in ((0, 1) if bs and not name.endswith("norm") else (0,)):
            assert (mapped.tensor_host(name, which, np.uint8) == again.tensor_host(name, which, np.uint8)).all()
    mapped.close()
    prompt = O.synth_tokens(10, 11, lo=3, hi=1000)
    c1, c2 = lcu.Context(model, 32, 0.8), lcu.Context(again, 32, 0.8)
    assert run_tokens(c1, prompt, 6) == run_tokens(c2, prompt, 6)
    om = O.OracleModel(n_vocab=1000, dim=256, context_len=32, temperature=0.8, path=d)
    assert om.next_token(prompt) >= 0
    om.close()
    if R.available():
        h = R.lib().ref_model_load(d.encode(), None)
        assert h
        R.lib().ref_model_free(h)
    # truncated / missing files are I/O errors, not crashes
    os.truncate(os.path.join(d, "norm.weight__256"), 100)
    with pytest.raises(lcu.LcuError, match="expected 512 bytes"):
        lcu.Model.load(d)
    os.remove(os.path.join(d, "params"))
    with pytest.raises(lcu.LcuError, match="params"):
        lcu.Model.load(d)
    for c in (c1, c2):
        c.close()
    model.close()
    again.close()


def test_quantize_model_dir_matches_in_memory_quantizer(lcu, tmp_path):
    fp = lcu.Model.synthetic(block_size=0, seed=5, scale=0.08, **SMALL)
    src, dst = str(tmp_path / "fp16"), str(tmp_path / "q8")
    fp.save(src)
    lcu.check(lcu.lib.lcu_quantize_model_dir(src.encode(), dst.encode(), 128))
    q8 = lcu.Model.load(dst)
    mem = lcu.Model.synthetic(block_size=128, seed=5, scale=0.08, **SMALL)
    for name in ("output", "layers.0.feed_forward.w1"):
        for which in (0, 1):
            assert (q8.tensor_host(name, which, np.uint8) == mem.tensor_host(name, which, np.uint8)).all()
    assert q8.params()["q_type"] == 1 and q8.params()["block_size"] == 128
    for m in (fp, q8, mem):
        m.close()


@pytest.mark.skipif(not R.available(), reason="reference library not built")
@pytest.mark.parametrize("bs,u8_mode", [(0, 1), (128, 1), (128, 0)], indirect=["u8_mode"])
def test_small_model_against_reference_forward(lcu, bs, u8_mode):
    cfg = dict(dim=512, n_heads=4, n_layers=4, n_vocab=2000)
    model = lcu.Model.synthetic(block_size=bs, seed=1234, scale=0.06, **cfg)
    ctx = lcu.Context(model, context_len=128, temperature=0.8)
    ref = R.RefModel(lcu, model, 512, 256, 4, 4, 2000, 1e-6, bs, 128, 0.8, mtype=4)
    prompt = O.synth_tokens(32, 1234, lo=3, hi=2000)
    t, tr = ctx.next_token(prompt), ref.next_token(prompt)
    mine, theirs = [], []
    for step in range(48):
        p, pr = f32(ctx.probs()), f32(ref.probs())
        assert np.abs(p - pr).max() <= 0.03 * pr.max() + 1e-4, step
        mine.append(t)
        theirs.append(tr)
        t, tr = ctx.next_token([tr]), ref.next_token([tr])  # teacher-forced on the reference's token
    assert np.mean(np.array(mine) == np.array(theirs)) >= 0.95, (mine, theirs)
    ref.close()
    ctx.close()
    model.close()
