"""The 7B-shaped configurations at full size: greedy tokens of the new library against the tokens the
reference itself produced on a B200 (tests/golden/reference_7b_tokens.json), fp16 and int8.

Batch-1 greedy decoding of a random-init model is chaotic: the reference's own two kernel sets
(matmul_type 4 vs 1) part ways after 13 steps on this input, because a different fp32 summation order
moves logits by an fp16 ulp and top-2 probability margins are often that small.  Where the free run leaves
the reference's is therefore luck (31 steps with one tiling of the prompt GEMMs, 12 with another); what the
test pins is what is stable: the free run may part only at a step where the reference itself is undecided
(top-1 / top-2 margin of a few fp16 ulps of its own probabilities), teacher-forced top-1 agreement is high,
and every teacher-forced disagreement sits at such a margin too."""
import json
import os

import numpy as np
import pytest

import oracle_lib as O

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_7b_tokens.json")))
CFG = dict(dim=4096, n_heads=32, n_layers=32, n_vocab=32000)


@pytest.fixture
def u8_mode(lcu, request):
    lcu.check(lcu.lib.lcu_set_tuning(b"int8_factored", request.param))
    yield request.param
    lcu.check(lcu.lib.lcu_set_tuning(b"int8_factored", 1))


@pytest.mark.parametrize("bs,u8_mode", [(0, 1), (128, 1), (128, 0)], indirect=["u8_mode"])
def test_7b_tokens_against_reference(lcu, bs, u8_mode, record_property):
    """u8_mode 1 = the default decode GEMV (scale factored out per block), 0 = the reference's per-weight rounding."""
    ref = np.array(GOLD[f"tokens_bs{bs}_t4"])
    margin = np.array(GOLD[f"top1_bs{bs}_t4"]) - np.array(GOLD[f"top2_bs{bs}_t4"])
    prompt = O.synth_tokens(128, 1234)
    model = lcu.Model.synthetic(block_size=bs, seed=1234, scale=0.02, **CFG)
    ctx = lcu.Context(model, 512, 0.8)
    first = ctx.next_token(prompt)
    chained, _ = ctx.decode_chained(first, 256)
    free = np.concatenate([[first], chained])
    diverge = int(np.argmax(free != ref)) if (free != ref).any() else len(ref)
    # (the reference's own matmul_type 1 leaves its matmul_type 4 after 13 steps on the fp16 model)
    assert diverge >= 4, diverge
    if diverge < len(ref):
        assert margin[diverge] <= 5e-4, (diverge, margin[diverge])
    ctx.clear_tokens()
    forced = [ctx.next_token(prompt)]
    for i in range(256):
        forced.append(ctx.next_token([int(ref[i])]))
    agree = np.array(forced) == ref
    # the figures a regression would move: where the free run leaves the reference's, and the teacher-forced agreement
    print(f"7B bs={bs} int8_factored={u8_mode}: free run identical for {diverge} steps (reference margin there "
          f"{margin[diverge] if diverge < len(ref) else float('nan'):.2e}), teacher-forced top-1 agreement {int(agree.sum())}/{len(agree)}")
    record_property("free_run_steps", diverge)
    record_property("teacher_forced_agreement", f"{int(agree.sum())}/{len(agree)}")
    assert agree.mean() >= 0.95, agree.mean()
    assert (margin[~agree] <= 5e-4).all(), margin[~agree]  # median margin is 1.2e-3; mismatches only where the reference itself is undecided
    # determinism: the chained run repeats bit for bit
    ctx.clear_tokens()
    assert ctx.next_token(prompt) == first
    again, _ = ctx.decode_chained(first, 256)
    assert (again == chained).all()
    ctx.close()
    model.close()


def test_7b_int8_top1_agreement_with_fp16(lcu):
    """Top-1 agreement of the quantized model with the fp16 model, teacher-forced on the fp16 run."""
    prompt = O.synth_tokens(128, 1234)
    runs = {}
    for bs in (0, 128):
        model = lcu.Model.synthetic(block_size=bs, seed=1234, scale=0.02, **CFG)
        ctx = lcu.Context(model, 512, 0.8)
        if bs == 0:
            t = ctx.next_token(prompt)
            toks = [t]
            for _ in range(64):
                t = ctx.next_token([t])
                toks.append(t)
            runs[0] = toks
        else:
            toks = [ctx.next_token(prompt)]
            for i in range(64):
                toks.append(ctx.next_token([runs[0][i]]))
            runs[128] = toks
        ctx.close()
        model.close()
    agree = np.mean(np.array(runs[0]) == np.array(runs[128]))
    # a reported figure, not a bar: random-init logits are nearly flat and the quantization error moves many argmaxes
    # (measured 0.58 .. 0.65, moving by a token or two with the summation order of the prompt kernels)
    print(f"top-1 agreement of the u8 model with the fp16 model over 65 teacher-forced steps: {agree:.3f}")
    assert agree >= 0.5, agree
