"""The CPU oracle against golden vectors produced by the reference itself on a B200
(tests/golden/reference_small.npz, written by tests/golden/make_golden.py).  No GPU needed."""
import os
import sys

import numpy as np
import pytest

import oracle_lib as O

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden as MG  # noqa: E402  (input generators only; nothing below touches a GPU)

L = O.lib()
G = np.load(os.path.join(HERE, "golden", "reference_small.npz"))


def f32(u):
    return np.asarray(u, np.uint16).view(np.float16).astype(np.float32)


def ulp_diff(a, b):
    return np.abs(a.astype(np.int32) - b.astype(np.int32))


@pytest.mark.parametrize("bs", [128, 64, 32])
def test_quantizer_bit_exact_with_reference(bs):
    x = MG.inputs_quant()
    q, s = O.quantize(x, 64, 512, bs)
    assert (s == G[f"quant_s_{bs}"]).all()
    assert (q == G[f"quant_q_{bs}"]).all()
    dq = np.empty_like(x)
    L.orc_dequantize_absmax_uint8(dq, s, q, 64, 512, bs)
    assert (dq == G[f"quant_dq_{bs}"]).all()
    st = np.zeros(3, np.float32)
    L.orc_error_stats(st, x.reshape(-1), dq.reshape(-1), x.size)
    assert np.allclose(st, G[f"quant_stats_{bs}"], rtol=2e-3, atol=1e-9)  # the reference sums with float atomics


def test_matmul_bit_exact_with_reference_naive_kernels():
    x, w, prev = MG.inputs_matmul()
    m, k, n = 3, 512, 128
    o = np.zeros((m, n), np.uint16)
    L.orc_matmul_nt_f16(o.reshape(-1), x.reshape(-1), w.reshape(-1), m, k, n, 0.0, 0)
    assert (o == G["mm_f16_t1"]).all()  # same sequential fp32 sum as llama_cu.cu:111-122
    o2 = prev.copy()
    L.orc_matmul_nt_f16(o2.reshape(-1), x.reshape(-1), w.reshape(-1), m, k, n, 1.0, 0)
    assert (o2 == G["mm_f16_beta_t1"]).all()
    q, s = O.quantize(w, n, k, 128)
    o3 = np.zeros((m, n), np.uint16)
    L.orc_matmul_nt_fp16u8(o3.reshape(-1), x.reshape(-1), q.reshape(-1), s.reshape(-1), m, k, n, 128, 0.0, 1)
    assert (o3 == G["mm_u8_t1"]).all()  # double products, float running sum (llama_cu.cu:125-145)


def test_matmul_close_to_reference_tensor_core_kernels():
    x, w, prev = MG.inputs_matmul()
    m, k, n = 3, 512, 128
    o = np.zeros((m, n), np.uint16)
    L.orc_matmul_nt_f16(o.reshape(-1), x.reshape(-1), w.reshape(-1), m, k, n, 0.0, 0)
    assert ulp_diff(o, G["mm_f16_t4"]).max() <= 2 and (o != G["mm_f16_t4"]).mean() < 0.1  # other summation order only
    q, s = O.quantize(w, n, k, 128)
    o3 = np.zeros((m, n), np.uint16)
    L.orc_matmul_nt_fp16u8(o3.reshape(-1), x.reshape(-1), q.reshape(-1), s.reshape(-1), m, k, n, 128, 0.0, 0)
    assert np.abs(f32(o3) - f32(G["mm_u8_t4"])).max() <= 4e-3
    assert (o3 != G["mm_u8_t4"]).mean() < 0.1


def test_row_kernels_against_reference():
    io = MG.inputs_ops()
    o = np.zeros_like(io["x"])
    L.orc_rms_norm(o.reshape(-1), io["x"].reshape(-1), io["nw"], 4, 512, 1e-6)
    d = ulp_diff(o, G["rms_norm"])
    assert d.max() <= 1 and (d > 0).mean() < 0.02  # rsqrtf: libm 1/sqrtf vs the device intrinsic
    o = np.zeros_like(io["a"])
    L.orc_silu(o, io["a"], io["b"], io["a"].size)
    d = ulp_diff(o, G["silu"])
    assert d.max() <= 1 and (d > 0).mean() < 0.02  # expf
    o = np.zeros_like(io["rot"])
    L.orc_rotary(o.reshape(-1), io["rot"].reshape(-1), 5, 256, 2, 7, 10000.0)
    assert np.abs(f32(o) - f32(G["rotary_pos7"])).max() <= 2e-3  # powf / sinf / cosf
    assert (o != G["rotary_pos7"]).mean() < 0.05


def test_attention_chain_against_reference():
    io = MG.inputs_ops()
    o = np.zeros_like(io["q"])
    L.orc_attention(o.reshape(-1), io["q"].reshape(-1), io["k"].reshape(-1), io["v"].reshape(-1), 1, 21, 256, 2, 20, 0)
    d = ulp_diff(o, G["attention_decode"])
    assert d.max() <= 2 and (d > 0).mean() < 0.05  # same sequential sums; expf ulps only
    o = np.zeros_like(io["q4"])
    L.orc_attention(o.reshape(-1), io["q4"].reshape(-1), io["k4"].reshape(-1), io["v4"].reshape(-1), 4, 4, 256, 2, 0, 0)
    d = ulp_diff(o, G["attention_prefill"])
    assert d.max() <= 2 and (d > 0).mean() < 0.05


@pytest.mark.parametrize("bs,mtype", [(0, 1), (0, 4), (128, 1), (128, 4)])
def test_forward_pass_against_reference_next_token(bs, mtype):
    """Greedy tokens and probabilities of the reference's own llama_context::next_token on a small model."""
    om = O.OracleModel(dim=256, multiple_of=256, n_heads=2, n_layers=3, n_vocab=1000, block_size=bs, seed=1234, scale=MG.SMALL_SCALE,
                       context_len=MG.SMALL_CTX, temperature=0.8)
    om.set_modes(wmma_rounding=1 if mtype == 4 else 0)
    prompt = O.synth_tokens(MG.SMALL_PROMPT, 1234, lo=3, hi=1000)
    want = G[f"fwd_tokens_bs{bs}_t{mtype}"]
    probs = G[f"fwd_probs_bs{bs}_t{mtype}"]
    got = [om.next_token(prompt)]
    assert np.abs(f32(om.probs()) - f32(probs[0])).max() <= 0.02 * f32(probs[0]).max() + 1e-5
    for i in range(MG.SMALL_STEPS):
        got.append(om.next_token([int(want[i])]))  # teacher-forced on the reference's own tokens
        if i == 0:
            assert np.abs(f32(om.probs()) - f32(probs[1])).max() <= 0.02 * f32(probs[1]).max() + 1e-5
    assert np.abs(f32(om.probs()) - f32(probs[2])).max() <= 0.02 * f32(probs[2]).max() + 1e-5
    agree = (np.array(got) == want).mean()
    assert agree >= (0.95 if mtype == 1 else 0.9), (got, want.tolist())
    om.close()
