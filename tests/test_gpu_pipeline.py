"""Layer pipeline over several GPUs (reference: partition / hop logic, llama_cu.cu:1114-1160): the same model
split over 2 (and 4) GPUs must emit exactly the tokens of the single-GPU run - the kernels are the same and
the hops copy activations verbatim, so the comparison is bit exact."""
import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu

CFG = dict(dim=512, n_heads=4, n_layers=8, n_vocab=2000, multiple_of=256)


def run_tokens(ctx, prompt, steps):
    toks = [ctx.next_token(prompt)]
    for _ in range(steps):
        toks.append(ctx.next_token([toks[-1]]))
    return toks


def split(n_layers, n_gpus):
    per = (n_layers + n_gpus - 1) // n_gpus
    return [min(i // per, n_gpus - 1) for i in range(n_layers)]


@pytest.mark.parametrize("n_gpus", [2, 4])
@pytest.mark.parametrize("bs", [0, 128])
def test_pipeline_equals_single_gpu(lcu, n_gpus, bs):
    if lcu.lib.lcu_device_count() < n_gpus:
        pytest.skip(f"needs {n_gpus} GPUs")
    prompt = O.synth_tokens(70, 77, lo=3, hi=2000)  # more than 64 rows: prompt GEMM and tiled attention on every stage
    outs = []
    for layer_gpus in (None, split(CFG["n_layers"], n_gpus)):
        model = lcu.Model.synthetic(block_size=bs, seed=4321, scale=0.06, layer_gpus=layer_gpus, **CFG)
        ctx = lcu.Context(model, context_len=128, temperature=0.8)
        toks = run_tokens(ctx, prompt, 24)
        chained, _ = ctx.decode_chained(toks[-1], 16)  # device-chained steps (CUDA graph on one GPU, stream-ordered hops on several)
        probs = ctx.probs().copy()
        outs.append((toks, list(chained), probs))
        ctx.close()
        model.close()
    assert outs[0][0] == outs[1][0]
    assert outs[0][1] == outs[1][1]
    assert (outs[0][2] == outs[1][2]).all()


def test_partition_helpers(lcu):
    import ctypes as C
    out = (C.c_int * 8)()
    assert lcu.lib.lcu_partition_even(8, 2, out) == 0
    assert list(out) == [0, 0, 0, 0, 1, 1, 1, 1]
