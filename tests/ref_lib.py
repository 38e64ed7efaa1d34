"""ctypes binding of the reference built for sm_100a (oracle/_ref/libllama_cu_ref.so).

Test infrastructure only: drives the reference's own kernels and its own forward pass on a GPU.
The library is built by `make -C oracle ref` where the reference sources are present; on a GPU
machine the prebuilt file is used.  `available()` is False when the file is absent.
"""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "oracle", "_ref", "libllama_cu_ref.so")
PATH_CUBLAS = os.path.join(ROOT, "oracle", "_ref", "libllama_cu_ref_cublas.so")  # the ENABLE_CUBLAS build: adds matmul_type 0
_LIB = None
_LIBS = {}
vp = C.c_void_p
u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
i16p = np.ctypeslib.ndpointer(np.int16, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


def available():
    return os.path.exists(PATH)


def cublas_available():
    return os.path.exists(PATH_CUBLAS)


def lib(cublas=False):
    """The reference library; cublas=True loads the variant built with ENABLE_CUBLAS (a separate copy with its own state)."""
    global _LIB
    if cublas:
        if "cublas" not in _LIBS:
            _LIBS["cublas"] = _bind(C.CDLL(PATH_CUBLAS))
        return _LIBS["cublas"]
    if _LIB is None:
        _LIB = _bind(C.CDLL(PATH))
    return _LIB


def _bind(L):
    sig = {
        "ref_initialize": (None, []),
        "ref_matmul_nt_f16": (C.c_int, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, vp]),
        "ref_matmul_nt_fp16u8": (C.c_int, [u16p, u16p, u8p, u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, vp]),
        "ref_matmul_rotating_ms": (C.c_float, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
        "ref_rms_norm": (C.c_int, [u16p, u16p, u16p, C.c_int, C.c_int, C.c_float]),
        "ref_rotary": (C.c_int, [u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int]),
        "ref_silu": (C.c_int, [u16p, u16p, u16p, C.c_size_t]),
        "ref_attention": (C.c_int, [u16p, u16p, u16p, u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
        "ref_model_alloc": (vp, [C.c_uint32] * 5 + [C.c_float, C.c_int, vp]),
        "ref_model_tensor": (C.c_int, [vp, C.c_char_p, C.c_int, C.POINTER(vp), C.POINTER(C.c_uint64)]),
        "ref_model_load": (vp, [C.c_char_p, vp]),
        "ref_model_fill_synthetic": (C.c_int, [vp, C.c_uint64, C.c_float]),
        "ref_tokenize": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int, i16p, C.c_int]),
        "ref_model_free": (None, [vp]),
        "ref_context_create": (vp, [vp, C.c_int, C.c_float, C.c_int]),
        "ref_context_free": (None, [vp]),
        "ref_context_clear": (None, [vp]),
        "ref_context_memory_usage": (C.c_uint64, [vp]),
        "ref_next_token": (C.c_int, [vp, i16p, C.c_int, C.c_int]),
        "ref_get_probs": (C.c_int, [vp, u16p]),
        "ref_decode_timed": (C.c_double, [vp, C.c_int16, C.c_int, i16p, C.c_int]),
        "ref_quantize_absmax_uint8": (C.c_int, [u8p, u16p, u16p, C.c_uint64, C.c_uint64, C.c_int, vp]),
        "ref_quantize_device": (C.c_int, [vp, vp, vp, C.c_uint64, C.c_uint64, C.c_int]),
        "ref_dequantize_absmax_uint8": (C.c_int, [u16p, u16p, u8p, C.c_uint64, C.c_uint64, C.c_int]),
        "ref_transform_quantize": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    return L


def matmul_f16(lhs, rhs, beta=0.0, out=None, mtype=4):
    m, k = lhs.shape
    n = rhs.shape[0]
    o = np.zeros((m, n), np.uint16) if out is None else np.ascontiguousarray(out).copy()
    assert lib().ref_matmul_nt_f16(o, np.ascontiguousarray(lhs), np.ascontiguousarray(rhs), m, k, n, beta, mtype, 0, None) == 0
    return o


def matmul_u8(lhs, q, scales, bs, beta=0.0, out=None, mtype=4):
    m, k = lhs.shape
    n = q.shape[0]
    o = np.zeros((m, n), np.uint16) if out is None else np.ascontiguousarray(out).copy()
    assert lib().ref_matmul_nt_fp16u8(o, np.ascontiguousarray(lhs), np.ascontiguousarray(q), np.ascontiguousarray(scales), m, k, n, bs,
                                      beta, mtype, 0, None) == 0
    return o


def quantize(w, bs):
    h, wd = w.shape
    q = np.empty((h, wd), np.uint8)
    s = np.empty((h, wd // bs), np.uint16)
    st = np.zeros(3, np.float32)
    assert lib().ref_quantize_absmax_uint8(q, s, np.ascontiguousarray(w), h, wd, bs, st.ctypes.data_as(vp)) == 0
    return q, s, st


TENSOR_NAMES_LAYER = ["attention_norm", "ffn_norm", "attention.wq", "attention.wk", "attention.wv", "attention.wo",
                      "feed_forward.w1", "feed_forward.w2", "feed_forward.w3"]


def tensor_names(n_layers):
    names = ["tok_embeddings", "output", "norm"]
    for i in range(n_layers):
        names += [f"layers.{i}.{t}" for t in TENSOR_NAMES_LAYER]
    return names


class RefModel:
    """The reference's llama_model_impl + llama_context_impl, weights copied on the device from a
    model of the new library (same bits on both sides, no files involved)."""

    def __init__(self, new_lib, new_model, dim, multiple_of, n_heads, n_layers, n_vocab, norm_eps, block_size,
                 context_len, temperature, mtype=4, layer_gpus=None):
        L = lib()
        self.mtype = mtype
        self.n_vocab = n_vocab
        lg = None if layer_gpus is None else np.ascontiguousarray(layer_gpus, np.int32).ctypes.data_as(vp)
        self.model = L.ref_model_alloc(dim, multiple_of, n_heads, n_layers, n_vocab, norm_eps, block_size, lg)
        assert self.model
        for name in tensor_names(n_layers):
            kinds = [0] if (block_size == 0 or name.endswith("norm")) else [0, 1]
            for which in kinds:
                dst, nb = vp(), C.c_uint64()
                assert L.ref_model_tensor(self.model, name.encode(), which, C.byref(dst), C.byref(nb)) == 0, name
                src, sb, _ = new_model.tensor(name, which)
                assert sb == nb.value, (name, which, sb, nb.value)
                assert new_lib.lib.lcu_memcpy_d2d(dst, vp(src), sb) == 0  # device-to-device, same bits on both sides
        self.ctx = L.ref_context_create(self.model, context_len, temperature, mtype)

    def next_token(self, tokens):
        t = np.ascontiguousarray(np.asarray(tokens, np.int16))
        return lib().ref_next_token(self.ctx, t, len(t), self.mtype)

    def probs(self):
        out = np.empty(self.n_vocab, np.uint16)
        assert lib().ref_get_probs(self.ctx, out) == 0
        return out

    def decode_timed(self, first, n):
        toks = np.empty(n, np.int16)
        secs = lib().ref_decode_timed(self.ctx, int(first), n, toks, self.mtype)
        return toks, secs

    def clear(self):
        lib().ref_context_clear(self.ctx)

    def close(self):
        L = lib()
        if self.ctx:
            L.ref_context_free(self.ctx)
            self.ctx = None
        if self.model:
            L.ref_model_free(self.model)
            self.model = None
