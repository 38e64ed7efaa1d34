"""Generates the golden vectors under tests/golden/ by running the REFERENCE ITSELF on a B200.

    python tests/golden/make_golden.py <output-dir>        # on a machine with a B200 and oracle/_ref built

The reference (eiz/llama.cu) ships no tests or golden vectors, so its own kernels and its own
llama_context::next_token - compiled unmodified for sm_100a into oracle/_ref/libllama_cu_ref.so -
are run on seeded inputs and the outputs are stored.  Inputs are not stored: they come from the
seeded generator (oracle_lib.synth_f16 / numpy default_rng), which the tests re-create.
tests/test_golden_cpu.py then checks the CPU oracle against these files without a GPU.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as O  # noqa: E402
import ref_lib as R  # noqa: E402
from conftest import load_package  # noqa: E402


def f16(a):
    return np.asarray(a, np.float32).astype(np.float16).view(np.uint16)


def inputs_quant():
    x = O.synth_f16(64 * 512, 1234, "golden.quant", 0.02).reshape(64, 512).copy()
    x[1, :128] = 0
    x[2, :] = f16(np.linspace(-3, 3, 512))
    x[3, :128] = 0x0001
    x[4, 128:256] = f16(np.arange(-64, 64) * 2.0 ** -7)
    return x


def inputs_matmul():
    rng = np.random.default_rng(2024)
    x = f16(rng.standard_normal((3, 512)))
    w = O.synth_f16(128 * 512, 1234, "golden.matmul", 0.05).reshape(128, 512)
    prev = f16(rng.standard_normal((3, 128)))
    return x, w, prev


def inputs_ops():
    rng = np.random.default_rng(2025)
    return dict(x=f16(rng.standard_normal((4, 512)) * 2), nw=f16(1 + 0.1 * rng.standard_normal(512)),
                a=f16(rng.standard_normal(768) * 3), b=f16(rng.standard_normal(768)),
                q=f16(rng.standard_normal((1, 256))), k=f16(rng.standard_normal((21, 256))), v=f16(rng.standard_normal((21, 256))),
                q4=f16(rng.standard_normal((4, 256))), k4=f16(rng.standard_normal((4, 256))), v4=f16(rng.standard_normal((4, 256))),
                rot=f16(rng.standard_normal((5, 256))))


SMALL = dict(dim=256, n_heads=2, n_layers=3, n_vocab=1000)
SMALL_SCALE, SMALL_CTX, SMALL_PROMPT, SMALL_STEPS = 0.08, 64, 12, 24


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    lcu = load_package()
    L = R.lib()
    g = {}
    # ---- quantizer (transform.cu:28-87)
    x = inputs_quant()
    for bs in (128, 64, 32):
        q, s, st = R.quantize(x, bs)
        dq = np.zeros_like(x)
        assert L.ref_dequantize_absmax_uint8(dq, s, q, 64, 512, bs) == 0
        g[f"quant_q_{bs}"], g[f"quant_s_{bs}"], g[f"quant_stats_{bs}"], g[f"quant_dq_{bs}"] = q, s, st, dq
    # ---- matmul_nt (llama_cu.cu:111-145 type 1, 225-366 type 4)
    xa, w, prev = inputs_matmul()
    q, s, _ = R.quantize(w, 128)
    for mtype in (1, 4):
        g[f"mm_f16_t{mtype}"] = R.matmul_f16(xa, w, mtype=mtype)
        g[f"mm_f16_beta_t{mtype}"] = R.matmul_f16(xa, w, beta=1.0, out=prev, mtype=mtype)
        g[f"mm_u8_t{mtype}"] = R.matmul_u8(xa, q, s, 128, mtype=mtype)
    # ---- row-wise kernels
    io = inputs_ops()
    o = np.zeros_like(io["x"])
    assert L.ref_rms_norm(o, io["x"], io["nw"], 4, 512, 1e-6) == 0
    g["rms_norm"] = o
    o = np.zeros_like(io["a"])
    assert L.ref_silu(o, io["a"], io["b"], io["a"].size) == 0
    g["silu"] = o
    o = np.zeros_like(io["rot"])
    assert L.ref_rotary(o, io["rot"], 5, 256, 2, 7) == 0
    g["rotary_pos7"] = o
    o = np.zeros_like(io["q"])
    assert L.ref_attention(o, io["q"], io["k"], io["v"], 1, 21, 256, 2, 20) == 0
    g["attention_decode"] = o
    o = np.zeros_like(io["q4"])
    assert L.ref_attention(o, io["q4"], io["k4"], io["v4"], 4, 4, 256, 2, 0) == 0
    g["attention_prefill"] = o
    # ---- forward pass of a small model through the reference's llama_context::next_token
    prompt = O.synth_tokens(SMALL_PROMPT, 1234, lo=3, hi=SMALL["n_vocab"])
    for bs in (0, 128):
        model = lcu.Model.synthetic(block_size=bs, seed=1234, scale=SMALL_SCALE, **SMALL)
        for mtype in (1, 4):
            ref = R.RefModel(lcu, model, SMALL["dim"], 256, SMALL["n_heads"], SMALL["n_layers"], SMALL["n_vocab"], 1e-6, bs, SMALL_CTX, 0.8,
                             mtype=mtype)
            toks = [ref.next_token(prompt)]
            probs = [ref.probs()]
            for _ in range(SMALL_STEPS):
                toks.append(ref.next_token([toks[-1]]))
                probs.append(ref.probs())
            g[f"fwd_tokens_bs{bs}_t{mtype}"] = np.array(toks, np.int16)
            g[f"fwd_probs_bs{bs}_t{mtype}"] = np.stack(probs)[[0, 1, SMALL_STEPS]]
            ref.close()
        model.close()
    np.savez_compressed(os.path.join(out_dir, "reference_small.npz"), **g)

    # ---- the 7B-shaped configurations: greedy tokens and top-2 probability margins of the reference
    big = {}
    cfg7 = dict(dim=4096, n_heads=32, n_layers=32, n_vocab=32000)
    prompt = O.synth_tokens(128, 1234)
    for bs, steps_by_type in ((0, {4: 256, 1: 48}), (128, {4: 256})):
        model = lcu.Model.synthetic(block_size=bs, seed=1234, scale=0.02, **cfg7)
        for mtype, steps in steps_by_type.items():
            ref = R.RefModel(lcu, model, 4096, 256, 32, 32, 32000, 1e-6, bs, 512, 0.8, mtype=mtype)
            toks, top1, top2 = [ref.next_token(prompt)], [], []
            for i in range(steps + 1):
                p = ref.probs().view(np.float16).astype(np.float32)
                part = np.partition(p, -2)[-2:]
                top1.append(float(part[1]))
                top2.append(float(part[0]))
                if i < steps:
                    toks.append(ref.next_token([toks[-1]]))
            big[f"tokens_bs{bs}_t{mtype}"] = [int(t) for t in toks]
            big[f"top1_bs{bs}_t{mtype}"] = top1
            big[f"top2_bs{bs}_t{mtype}"] = top2
            ref.close()
        model.close()
    json.dump(big, open(os.path.join(out_dir, "reference_7b_tokens.json"), "w"))
    print("golden vectors written to", out_dir)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
