"""Tensor-parallel decode (lcu_tp_*): every GPU streams its own rows of every matrix and the slices of the activation rows
travel as peer stores from the GEMV epilogues.  Each output element is computed by the same kernel code in the same order
as on one GPU, so tokens AND probabilities must be bit-identical to a single-GPU context fed the same tokens one at a
time (a prompt runs as single-token steps in the tensor-parallel decoder)."""
import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu

TINY = dict(dim=512, n_heads=4, n_layers=4, n_vocab=2000)


def single_gpu_run(lcu, cfg, bs, prompt, steps, chained, seed, scale, ctx_len):
    model = lcu.Model.synthetic(block_size=bs, seed=seed, scale=scale, **cfg)
    ctx = lcu.Context(model, context_len=ctx_len, temperature=0.8)
    t = None
    for tok in prompt:  # token by token: the decode kernels, like the tensor-parallel decoder's prompt
        t = ctx.next_token([int(tok)])
    toks = [t]
    for _ in range(steps):
        toks.append(ctx.next_token([toks[-1]]))
    probs = ctx.probs().copy()
    ch, _ = ctx.decode_chained(toks[-1], chained)
    ctx.close()
    return model, toks, probs, list(ch)


@pytest.mark.parametrize("n_gpus", [2, 4])
@pytest.mark.parametrize("bs", [0, 128])
def test_tensor_parallel_equals_single_gpu(lcu, tmp_path, n_gpus, bs):
    if lcu.lib.lcu_device_count() < n_gpus:
        pytest.skip(f"needs {n_gpus} GPUs")
    prompt = O.synth_tokens(9, 77, lo=3, hi=2000)
    model, toks, probs, chained = single_gpu_run(lcu, TINY, bs, prompt, 12, 8, 4321, 0.06, 128)
    tp = lcu.TensorParallel(n_gpus, block_size=bs, context_len=128, temperature=0.8, seed=4321, scale=0.06, **TINY)
    mine = [tp.next_token(prompt)]
    for _ in range(12):
        mine.append(tp.next_token([mine[-1]]))
    assert mine == toks
    assert (tp.probs() == probs).all()
    ch, ms = tp.decode_chained(mine[-1], 8)
    assert list(ch) == chained and ms > 0
    assert tp.tokens_left() == 128 - 9 - 12 - 8
    # the same model from a weight directory: every GPU reads its rows of every file
    d = str(tmp_path / "m")
    model.save(d)
    model.close()
    tp2 = lcu.TensorParallel(n_gpus, block_size=bs, context_len=128, temperature=0.8, path=d, **TINY)
    assert tp2.next_token(prompt) == toks[0]
    tp2.close()
    # a second conversation on the same decoder (the flag numbering carries on)
    tp.clear_tokens()
    assert tp.next_token(prompt) == toks[0]
    assert tp.weight_bytes_per_gpu() > 0
    tp.close()


@pytest.mark.parametrize("dim,n_heads,bs", [(8192, 64, 128), (5120, 40, 0)])
def test_tensor_parallel_at_large_widths(lcu, dim, n_heads, bs):
    """One layer at the 65B (u8) and 13B (fp16) widths over 2 GPUs: the shapes the sharded GEMVs run in the benchmark."""
    if lcu.lib.lcu_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cfg = dict(dim=dim, n_heads=n_heads, n_layers=1, n_vocab=2000)
    prompt = O.synth_tokens(4, 5, lo=3, hi=2000)
    model, toks, probs, chained = single_gpu_run(lcu, cfg, bs, prompt, 4, 4, 99, 0.02, 32)
    model.close()
    tp = lcu.TensorParallel(2, block_size=bs, context_len=32, temperature=0.8, seed=99, scale=0.02, **cfg)
    mine = [tp.next_token(prompt)]
    for _ in range(4):
        mine.append(tp.next_token([mine[-1]]))
    assert mine == toks and (tp.probs() == probs).all()
    ch, _ = tp.decode_chained(mine[-1], 4)
    assert list(ch) == chained
    tp.close()


def test_tensor_parallel_rejects_bad_splits(lcu):
    raw = lcu.pack_params(512, 256, 4, 4, 2000)
    assert lcu.lib.lcu_tp_check_split(raw, 2) == 0 and lcu.lib.lcu_tp_check_split(raw, 4) == 0
    assert lcu.lib.lcu_tp_check_split(raw, 8) != 0 and b"heads" in lcu.lib.lcu_last_error()
    assert lcu.lib.lcu_tp_check_split(raw, 1) != 0


def test_tensor_parallel_as_the_first_work_of_a_process(lcu):
    """The CUDA runtime loads a kernel at its first launch, and that loading may wait for the device to go idle.  A
    tensor-parallel step whose launches stalled there, between a kernel that already waits and the launch it waits for,
    would run into the bounded waits.  The decoder therefore loads all kernels of a step when it is created; this runs it
    in a fresh process where nothing has been launched before."""
    import os
    import subprocess
    import sys
    if lcu.lib.lcu_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    code = ("import sys; sys.path.insert(0, %r); from conftest import load_package; lcu = load_package()\n"
            "tp = lcu.TensorParallel(2, dim=1024, n_heads=8, n_layers=6, n_vocab=32000, block_size=128, context_len=64, temperature=0.8, seed=3, scale=0.04)\n"
            "t = tp.next_token([5, 6, 7, 8]); ch, ms = tp.decode_chained(t, 8); print('ok', t, list(ch))\n") % here
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.startswith("ok"), (r.stdout[-500:], r.stderr[-1500:])
