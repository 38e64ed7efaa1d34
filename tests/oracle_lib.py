"""ctypes binding of the CPU oracle (oracle/liboracle.so).  Test infrastructure only."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB = None

u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
i16p = np.ctypeslib.ndpointer(np.int16, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = os.path.join(ROOT, "oracle", "liboracle.so")
    if not os.path.exists(path):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), path])
    L = C.CDLL(path)
    sig = {
        "orc_init": (None, []),
        "orc_f2h": (C.c_uint16, [C.c_float]),
        "orc_h2f": (C.c_float, [C.c_uint16]),
        "orc_fnv1a64": (C.c_uint64, [C.c_char_p]),
        "orc_synth_fill_f16": (None, [u16p, C.c_uint64, C.c_uint64, C.c_char_p, C.c_float, C.c_uint64]),
        "orc_synth_tokens": (None, [i16p, C.c_int, C.c_uint64, C.c_char_p, C.c_int, C.c_int]),
        "orc_quantize_absmax_uint8": (None, [u8p, u16p, u16p, C.c_uint64, C.c_uint64, C.c_int]),
        "orc_dequantize_absmax_uint8": (None, [u16p, u16p, u8p, C.c_uint64, C.c_uint64, C.c_int]),
        "orc_error_stats": (None, [f32p, u16p, u16p, C.c_uint64]),
        "orc_matmul_nt_f16": (None, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]),
        "orc_matmul_nt_fp16u8": (None, [u16p, u16p, u8p, u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]),
        "orc_matmul_nt_gold": (None, [f64p, u16p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
        "orc_rms_norm": (None, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_float]),
        "orc_rotary": (None, [u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]),
        "orc_matmul_qk": (None, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
        "orc_softmax_rows": (None, [u16p, u16p, C.c_uint64, C.c_int, C.c_float]),
        "orc_matmul_qkv": (None, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int]),
        "orc_attention": (None, [u16p, u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
        "orc_silu": (None, [u16p, u16p, u16p, C.c_uint64]),
        "orc_matmul_nt_f16_gated": (None, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int]),
        "orc_ffn_dim": (C.c_uint32, [C.c_uint32, C.c_uint32]),
        "orc_model_create_synth": (C.c_void_p, [C.c_uint32] * 5 + [C.c_float, C.c_int, C.c_uint64, C.c_float]),
        "orc_model_load": (C.c_void_p, [C.c_char_p]),
        "orc_model_free": (None, [C.c_void_p]),
        "orc_context_create": (C.c_void_p, [C.c_void_p, C.c_int, C.c_float]),
        "orc_context_free": (None, [C.c_void_p]),
        "orc_context_clear": (None, [C.c_void_p]),
        "orc_context_set_modes": (None, [C.c_void_p, C.c_int, C.c_int]),
        "orc_context_pos": (C.c_int, [C.c_void_p]),
        "orc_next_token": (C.c_int, [C.c_void_p, i16p, C.c_int]),
        "orc_get_probs": (None, [C.c_void_p, u16p]),
        "orc_get_logits": (None, [C.c_void_p, u16p]),
        "orc_get_last_hidden": (None, [C.c_void_p, u16p]),
        "orc_sample_token": (C.c_int, [u16p, C.c_int, C.c_float]),
        "orc_sampler_uniform": (C.c_float, [C.c_uint64, C.c_int]),
        "orc_num_threads": (C.c_int, []),
        "orc_set_num_threads": (C.c_int, [C.c_int]),
        "orc_last_timing": (C.c_double, [C.c_void_p, C.c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    L.orc_init()
    _LIB = L
    return L


def synth_f16(n, seed, name, scale, first=0):
    out = np.empty(int(n), np.uint16)
    lib().orc_synth_fill_f16(out, int(n), seed, name.encode(), scale, first)
    return out


def synth_tokens(n, seed, name=b"prompt", lo=3, hi=32000):
    out = np.empty(n, np.int16)
    lib().orc_synth_tokens(out, n, seed, name if isinstance(name, bytes) else name.encode(), lo, hi)
    return out


def quantize(w_u16, h, w, bs):
    q = np.empty((h, w), np.uint8)
    s = np.empty((h, w // bs), np.uint16)
    lib().orc_quantize_absmax_uint8(q, s, np.ascontiguousarray(w_u16).reshape(-1), h, w, bs)
    return q, s


class OracleModel:
    """Synthetic or file-loaded model + one context, mirroring llama_model / llama_context."""

    def __init__(self, dim=None, multiple_of=256, n_heads=None, n_layers=None, n_vocab=None, norm_eps=1e-6,
                 block_size=0, seed=1234, scale=0.02, context_len=256, temperature=0.8, path=None):
        L = lib()
        if path is not None:
            self.model = L.orc_model_load(path.encode())
        else:
            self.model = L.orc_model_create_synth(dim, multiple_of, n_heads, n_layers, n_vocab, norm_eps, block_size, seed, scale)
        if not self.model:
            raise RuntimeError("oracle model could not be created")
        self.n_vocab = n_vocab
        self.dim = dim
        self.ctx = L.orc_context_create(self.model, context_len, temperature)

    def set_modes(self, wmma_rounding=1, fp32_attention=0):
        lib().orc_context_set_modes(self.ctx, wmma_rounding, fp32_attention)

    def clear(self):
        lib().orc_context_clear(self.ctx)

    def next_token(self, tokens):
        t = np.ascontiguousarray(np.asarray(tokens, np.int16))
        return lib().orc_next_token(self.ctx, t, len(t))

    def probs(self):
        out = np.empty(self.n_vocab, np.uint16)
        lib().orc_get_probs(self.ctx, out)
        return out

    def logits(self):
        out = np.empty(self.n_vocab, np.uint16)
        lib().orc_get_logits(self.ctx, out)
        return out

    def last_hidden(self):
        out = np.empty(self.dim, np.uint16)
        lib().orc_get_last_hidden(self.ctx, out)
        return out

    def close(self):
        L = lib()
        if self.ctx:
            L.orc_context_free(self.ctx)
            self.ctx = None
        if self.model:
            L.orc_model_free(self.model)
            self.model = None
