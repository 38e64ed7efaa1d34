"""ctypes binding of libllama_cu_b200.so (the C ABI declared in include/llama_cu_c.h).

The package directory name contains a dot, so it is loaded by path (see `load_package` in
tests/conftest.py and bench.py) under the module name ``llama_cu_b200``.  There is no CPU
fallback: importing works anywhere, but every compute call needs an sm_100a device, and a
missing shared library raises at import time.
"""
import ctypes as C
import os
import struct

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libllama_cu_b200.so")
if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
        "(or __graft_entry__.build()); this package has no CPU implementation"
    )
lib = C.CDLL(LIB_PATH)

vp = C.c_void_p
_SIG = {
    "lcu_last_error": (C.c_char_p, []),
    "lcu_initialize": (C.c_int, [C.c_int]),
    "lcu_device_count": (C.c_int, []),
    "lcu_set_matmul_type": (C.c_int, [C.c_int]),
    "lcu_set_tuning": (C.c_int, [C.c_char_p, C.c_int]),
    "lcu_malloc": (C.c_int, [C.POINTER(vp), C.c_uint64]),
    "lcu_free": (C.c_int, [vp]),
    "lcu_memcpy_h2d": (C.c_int, [vp, vp, C.c_uint64]),
    "lcu_memcpy_d2h": (C.c_int, [vp, vp, C.c_uint64]),
    "lcu_memcpy_d2d": (C.c_int, [vp, vp, C.c_uint64]),
    "lcu_memset": (C.c_int, [vp, C.c_int, C.c_uint64]),
    "lcu_mem_info": (C.c_int, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "lcu_partition_is_contiguous": (C.c_int, [vp, C.c_int]),
    "lcu_context_scratch_bytes": (C.c_uint64, [vp, C.c_int]),
    "lcu_context_kv_bytes_per_layer": (C.c_uint64, [vp, C.c_int]),
    "lcu_tokenize": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int, vp, C.c_int]),
    "lcu_set_device": (C.c_int, [C.c_int]),
    "lcu_synchronize": (C.c_int, []),
    "lcu_quantize_absmax_uint8": (C.c_int, [vp, vp, vp, C.c_uint64, C.c_uint64, C.c_int, vp]),
    "lcu_dequantize_absmax_uint8": (C.c_int, [vp, vp, vp, C.c_uint64, C.c_uint64, C.c_int, vp]),
    "lcu_error_stats": (C.c_int, [vp, vp, vp, C.c_uint64, vp]),
    "lcu_quantize_host": (C.c_int, [vp, vp, vp, C.c_uint64, C.c_uint64, C.c_int, vp]),
    "lcu_quantize_model_dir": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int]),
    "lcu_matmul_nt_f16": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_float, vp]),
    "lcu_matmul_nt_f16_gated": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "lcu_matmul_nt_fp16u8": (C.c_int, [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, vp]),
    "lcu_rms_norm": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_float, vp]),
    "lcu_silu": (C.c_int, [vp, vp, vp, C.c_uint64, vp]),
    "lcu_rope_scatter": (C.c_int, [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "lcu_rope_scatter_static": (C.c_int, [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "lcu_attention": (C.c_int, [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "lcu_logits_head": (C.c_int, [vp, vp, C.c_int, C.c_float, C.POINTER(C.c_int), vp]),
    "lcu_selftest_bounded_wait": (C.c_int, [C.POINTER(C.c_int)]),
    "lcu_selftest_quantizer_arithmetic": (C.c_int, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "lcu_selftest_balanced_schedule": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "lcu_plan_long_prompt_gemm": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]),
    "lcu_plan_short_prompt_gemm": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "lcu_selftest_silu_arithmetic": (C.c_int, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "lcu_bench_matmul_f16": (C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "lcu_synth_fill_f16": (C.c_int, [vp, C.c_uint64, C.c_uint64, C.c_char_p, C.c_float, C.c_uint64, vp]),
    "lcu_model_create": (C.c_int, [vp, vp, C.POINTER(vp)]),
    "lcu_model_load": (C.c_int, [C.c_char_p, vp, C.POINTER(vp)]),
    "lcu_model_fill_synthetic": (C.c_int, [vp, C.c_uint64, C.c_float]),
    "lcu_model_save": (C.c_int, [vp, C.c_char_p]),
    "lcu_model_tensor": (C.c_int, [vp, C.c_char_p, C.c_int, C.POINTER(vp), C.POINTER(C.c_uint64), C.POINTER(C.c_int)]),
    "lcu_model_params": (C.c_int, [vp, vp]),
    "lcu_model_weight_bytes": (C.c_uint64, [vp]),
    "lcu_model_shadow_bytes": (C.c_uint64, [vp]),
    "lcu_model_free": (None, [vp]),
    "lcu_ffn_dim": (C.c_uint32, [C.c_uint32, C.c_uint32]),
    "lcu_partition_autopipe": (C.c_int, [vp, C.c_int, vp]),
    "lcu_partition_even": (C.c_int, [C.c_int, C.c_int, vp]),
    "lcu_context_create": (C.c_int, [vp, C.c_int, C.c_float, C.POINTER(vp)]),
    "lcu_context_free": (None, [vp]),
    "lcu_context_clear_tokens": (None, [vp]),
    "lcu_context_memory_usage": (C.c_uint64, [vp]),
    "lcu_context_tokens_left": (C.c_int, [vp]),
    "lcu_context_next_token": (C.c_int, [vp, vp, C.c_int, C.POINTER(C.c_int)]),
    "lcu_context_decode_chained": (C.c_int, [vp, C.c_int16, C.c_int, vp, C.POINTER(C.c_float)]),
    "lcu_context_read_probs": (C.c_int, [vp, vp]),
    "lcu_context_read_hidden": (C.c_int, [vp, vp]),
    "lcu_context_kernels_per_step": (C.c_int, [vp]),
    "lcu_context_set_sampling": (C.c_int, [vp, C.c_int, C.c_uint64]),
    "lcu_context_rollover": (C.c_int, [vp, C.c_int]),
    "lcu_rollover": (C.c_int, [vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp]),
    "lcu_sampler_uniform": (C.c_float, [C.c_uint64, C.c_int]),
    "lcu_sample_token": (C.c_int, [vp, C.c_int, C.c_float, C.POINTER(C.c_int), vp]),
    "lcu_tp_check_split": (C.c_int, [vp, C.c_int]),
    "lcu_tp_create": (C.c_int, [vp, vp, C.c_int, C.c_int, C.c_float, C.POINTER(vp)]),
    "lcu_tp_fill_synthetic": (C.c_int, [vp, C.c_uint64, C.c_float]),
    "lcu_tp_load": (C.c_int, [vp, C.c_char_p]),
    "lcu_tp_next_token": (C.c_int, [vp, vp, C.c_int, C.POINTER(C.c_int)]),
    "lcu_tp_decode_chained": (C.c_int, [vp, C.c_int16, C.c_int, vp, C.POINTER(C.c_float)]),
    "lcu_tp_read_probs": (C.c_int, [vp, vp]),
    "lcu_tp_clear_tokens": (None, [vp]),
    "lcu_tp_tokens_left": (C.c_int, [vp]),
    "lcu_tp_kernels_per_step": (C.c_int, [vp]),
    "lcu_tp_weight_bytes_per_gpu": (C.c_uint64, [vp]),
    "lcu_tp_free": (None, [vp]),
    "lcu_bench_decode_kernel": (C.c_int, [vp, C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_uint64)]),
    "lcu_profiler_start": (C.c_int, []),
    "lcu_profiler_stop": (C.c_int, []),
    "lcu_bench_quantize": (C.c_int, [C.c_uint64, C.c_uint64, C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "lcu_bench_read_ceiling": (C.c_int, [C.c_uint64, C.c_int, C.c_int, C.POINTER(C.c_float)]),
}
EXPORTS = sorted(_SIG)
for _name, (_res, _args) in _SIG.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


class LcuError(RuntimeError):
    pass


def check(rc):
    if rc != 0:
        raise LcuError(f"status {rc}: {lib.lcu_last_error().decode(errors='replace')}")


PARAMS_FMT = "<QIIIIIIfBBH"  # the 40-byte params record
MAGIC = 0x000041524F525541
FOURCC = 0x414D4C4C


def pack_params(dim, multiple_of, n_heads, n_layers, n_vocab, norm_eps=1e-6, block_size=0):
    return struct.pack(PARAMS_FMT, MAGIC, FOURCC, dim, multiple_of, n_heads, n_layers, n_vocab, norm_eps,
                       1 if block_size else 0, 0, block_size)


def _ptr(a):
    return a.ctypes.data_as(vp)


class DeviceBuffer:
    """Plain device allocation (cudaMalloc) for callers that do not use torch."""

    def __init__(self, nbytes):
        self.ptr = vp()
        self.nbytes = int(nbytes)
        check(lib.lcu_malloc(C.byref(self.ptr), self.nbytes))

    @classmethod
    def from_host(cls, arr):
        arr = np.ascontiguousarray(arr)
        b = cls(max(arr.nbytes, 1))
        if arr.nbytes:
            check(lib.lcu_memcpy_h2d(b.ptr, _ptr(arr), arr.nbytes))
        return b

    def to_host(self, dtype, shape):
        out = np.empty(shape, dtype)
        if out.nbytes:
            check(lib.lcu_memcpy_d2h(_ptr(out), self.ptr, out.nbytes))
        return out

    def free(self):
        if self.ptr:
            lib.lcu_free(self.ptr)
            self.ptr = vp()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


# ---- host-array convenience wrappers (copy in, run on the GPU, copy out) ---------------------
def quantize(w_u16, bs, stats=False):
    """fp16 matrix (uint16 view, 2-D) -> (q uint8, scales uint16[, stats float32[3]])."""
    w = np.ascontiguousarray(w_u16, np.uint16)
    h, wd = w.shape
    q = np.empty((h, wd), np.uint8)
    s = np.empty((h, wd // bs), np.uint16)
    st = np.zeros(3, np.float32)
    check(lib.lcu_quantize_host(_ptr(q), _ptr(s), _ptr(w), h, wd, bs, _ptr(st) if stats else None))
    return (q, s, st) if stats else (q, s)


def dequantize(q, scales, bs):
    h, w = q.shape
    dq, ds, do = DeviceBuffer.from_host(q), DeviceBuffer.from_host(scales), DeviceBuffer(h * w * 2)
    check(lib.lcu_dequantize_absmax_uint8(do.ptr, ds.ptr, dq.ptr, h, w, bs, None))
    check(lib.lcu_synchronize())
    return do.to_host(np.uint16, (h, w))


def matmul_nt_gated(lhs_u16, w13_u16, tile=256):
    """silu(lhs . w1^T) * (lhs . w3^T) on half-rounded products as one launch; w13 = [w1; w3] stacked, (2 f, k)."""
    lhs = np.ascontiguousarray(lhs_u16, np.uint16)
    w13 = np.ascontiguousarray(w13_u16, np.uint16)
    m, k = lhs.shape
    f = w13.shape[0] // 2
    dl, dr, do = DeviceBuffer.from_host(lhs), DeviceBuffer.from_host(w13), DeviceBuffer.from_host(np.zeros((m, f), np.uint16))
    check(lib.lcu_matmul_nt_f16_gated(do.ptr, dl.ptr, dr.ptr, m, k, f, tile, None))
    check(lib.lcu_synchronize())
    return do.to_host(np.uint16, (m, f))


def matmul_nt(lhs_u16, rhs, scales=None, bs=0, beta=0.0, out_u16=None):
    """out(m,n) = lhs(m,k) . rhs(n,k)^T + beta*out; rhs fp16 (uint16 view) or uint8 with scales."""
    lhs = np.ascontiguousarray(lhs_u16, np.uint16)
    m, k = lhs.shape
    n = rhs.shape[0]
    out = np.zeros((m, n), np.uint16) if out_u16 is None else np.ascontiguousarray(out_u16, np.uint16).copy()
    dl, dr, do = DeviceBuffer.from_host(lhs), DeviceBuffer.from_host(rhs), DeviceBuffer.from_host(out)
    if scales is None:
        check(lib.lcu_matmul_nt_f16(do.ptr, dl.ptr, dr.ptr, m, k, n, beta, None))
    else:
        dsc = DeviceBuffer.from_host(scales)
        check(lib.lcu_matmul_nt_fp16u8(do.ptr, dl.ptr, dr.ptr, dsc.ptr, m, k, n, bs, beta, None))
    check(lib.lcu_synchronize())
    return do.to_host(np.uint16, (m, n))


def rms_norm(x_u16, weight_u16, eps):
    x = np.ascontiguousarray(x_u16, np.uint16)
    rows, dim = x.shape
    dx, dw, do = DeviceBuffer.from_host(x), DeviceBuffer.from_host(weight_u16), DeviceBuffer(x.nbytes)
    check(lib.lcu_rms_norm(do.ptr, dx.ptr, dw.ptr, rows, dim, eps, None))
    check(lib.lcu_synchronize())
    return do.to_host(np.uint16, (rows, dim))


def silu(a_u16, b_u16):
    a = np.ascontiguousarray(a_u16, np.uint16)
    da, db, do = DeviceBuffer.from_host(a), DeviceBuffer.from_host(b_u16), DeviceBuffer(a.nbytes)
    check(lib.lcu_silu(do.ptr, da.ptr, db.ptr, a.size, None))
    check(lib.lcu_synchronize())
    return do.to_host(np.uint16, a.shape)


def attention(q_u16, k_u16, v_u16, n_heads, start_pos, cluster=1):
    """Fused attention on row-major inputs: q (m,dim) rotated, k/v (T,dim) with T = start_pos + m and
    k already rotated.  Builds the head-major caches, runs the kernel, returns out (m,dim)."""
    q = np.ascontiguousarray(q_u16, np.uint16)
    m, dim = q.shape
    T = k_u16.shape[0]
    hd = dim // n_heads
    to_cache = lambda a: np.ascontiguousarray(np.asarray(a, np.uint16).reshape(T, n_heads, hd).transpose(1, 0, 2))
    dq, dk, dv = DeviceBuffer.from_host(q), DeviceBuffer.from_host(to_cache(k_u16)), DeviceBuffer.from_host(to_cache(v_u16))
    do = DeviceBuffer(q.nbytes)
    check(lib.lcu_attention(do.ptr, dq.ptr, dk.ptr, dv.ptr, start_pos, m, dim, n_heads, T, cluster, None))
    check(lib.lcu_synchronize())
    return do.to_host(np.uint16, (m, dim))


def rope_scatter(q_u16, k_new_u16, v_new_u16, n_heads, pos0, ctx_len):
    """Returns (rotated q (m,dim), k_cache, v_cache) with caches head-major (n_heads, ctx_len, hd)."""
    q = np.ascontiguousarray(q_u16, np.uint16)
    m, dim = q.shape
    hd = dim // n_heads
    dq, dk, dv = DeviceBuffer.from_host(q), DeviceBuffer.from_host(k_new_u16), DeviceBuffer.from_host(v_new_u16)
    kc, vc = DeviceBuffer(ctx_len * dim * 2), DeviceBuffer(ctx_len * dim * 2)
    check(lib.lcu_memset(kc.ptr, 0, kc.nbytes))
    check(lib.lcu_memset(vc.ptr, 0, vc.nbytes))
    check(lib.lcu_rope_scatter(dq.ptr, dk.ptr, dv.ptr, kc.ptr, vc.ptr, pos0, m, dim, n_heads, ctx_len, None))
    check(lib.lcu_synchronize())
    return (dq.to_host(np.uint16, (m, dim)), kc.to_host(np.uint16, (n_heads, ctx_len, hd)),
            vc.to_host(np.uint16, (n_heads, ctx_len, hd)))


def logits_head(logits_u16, temperature):
    lg = np.ascontiguousarray(logits_u16, np.uint16)
    dl, dp = DeviceBuffer.from_host(lg), DeviceBuffer(lg.nbytes)
    tok = C.c_int(0)
    check(lib.lcu_logits_head(dp.ptr, dl.ptr, lg.size, temperature, C.byref(tok), None))
    return tok.value, dp.to_host(np.uint16, lg.shape)


def synth_f16(n, seed, name, scale, first=0):
    d = DeviceBuffer(n * 2)
    check(lib.lcu_synth_fill_f16(d.ptr, n, seed, name.encode(), scale, first, None))
    check(lib.lcu_synchronize())
    return d.to_host(np.uint16, (n,))


class Model:
    """llama_model: weights on the GPU(s), from a weight directory or seeded synthetic data."""

    def __init__(self, handle, n_vocab, dim):
        self.handle, self.n_vocab, self.dim = handle, n_vocab, dim

    @classmethod
    def synthetic(cls, dim, n_heads, n_layers, n_vocab, multiple_of=256, norm_eps=1e-6, block_size=0, seed=1234,
                  scale=0.02, layer_gpus=None):
        h = vp()
        lg = None if layer_gpus is None else _ptr(np.ascontiguousarray(layer_gpus, np.int32))
        check(lib.lcu_model_create(pack_params(dim, multiple_of, n_heads, n_layers, n_vocab, norm_eps, block_size), lg, C.byref(h)))
        m = cls(h, n_vocab, dim)
        check(lib.lcu_model_fill_synthetic(h, seed, scale))
        return m

    @classmethod
    def load(cls, path, layer_gpus=None):
        h = vp()
        lg = None if layer_gpus is None else _ptr(np.ascontiguousarray(layer_gpus, np.int32))
        check(lib.lcu_model_load(path.encode(), lg, C.byref(h)))
        raw = C.create_string_buffer(40)
        lib.lcu_model_params(h, raw)
        f = struct.unpack(PARAMS_FMT, raw.raw)
        return cls(h, f[6], f[2])

    def params(self):
        raw = C.create_string_buffer(40)
        lib.lcu_model_params(self.handle, raw)
        keys = ("magic", "fourcc", "dim", "multiple_of", "n_heads", "n_layers", "n_vocab", "norm_eps", "q_type", "reserved0", "block_size")
        return dict(zip(keys, struct.unpack(PARAMS_FMT, raw.raw)))

    def tensor(self, name, which=0):
        p, b, d = vp(), C.c_uint64(), C.c_int()
        check(lib.lcu_model_tensor(self.handle, name.encode(), which, C.byref(p), C.byref(b), C.byref(d)))
        return p.value, b.value, d.value

    def tensor_host(self, name, which=0, dtype=np.uint16):
        p, b, _ = self.tensor(name, which)
        out = np.empty(b // np.dtype(dtype).itemsize, dtype)
        check(lib.lcu_memcpy_d2h(_ptr(out), p, b))
        return out

    def save(self, path):
        check(lib.lcu_model_save(self.handle, path.encode()))

    def weight_bytes(self):
        return lib.lcu_model_weight_bytes(self.handle)

    def shadow_bytes(self):
        """u8 models: bytes of the fp16 copy of the layer matrices kept for prompts (0 while there is none)."""
        return lib.lcu_model_shadow_bytes(self.handle)

    def close(self):
        if self.handle:
            lib.lcu_model_free(self.handle)
            self.handle = None


class Context:
    """llama_context: KV cache + forward pass.  next_token mirrors the reference's method."""

    def __init__(self, model, context_len=2048, temperature=0.9):
        self.model = model
        self.handle = vp()
        check(lib.lcu_context_create(model.handle, context_len, temperature, C.byref(self.handle)))

    def next_token(self, tokens):
        t = np.ascontiguousarray(np.asarray(tokens, np.int16))
        out = C.c_int(0)
        check(lib.lcu_context_next_token(self.handle, _ptr(t), len(t), C.byref(out)))
        return out.value

    def decode_chained(self, first_token, n_steps):
        toks = np.empty(n_steps, np.int16)
        ms = C.c_float(0)
        check(lib.lcu_context_decode_chained(self.handle, int(first_token), n_steps, _ptr(toks), C.byref(ms)))
        return toks, ms.value

    def clear_tokens(self):
        lib.lcu_context_clear_tokens(self.handle)

    def tokens_left(self):
        return lib.lcu_context_tokens_left(self.handle)

    def memory_usage(self):
        return lib.lcu_context_memory_usage(self.handle)

    def probs(self):
        out = np.empty(self.model.n_vocab, np.uint16)
        check(lib.lcu_context_read_probs(self.handle, _ptr(out)))
        return out

    def hidden(self):
        out = np.empty(self.model.dim, np.uint16)
        check(lib.lcu_context_read_hidden(self.handle, _ptr(out)))
        return out

    def kernels_per_step(self):
        return lib.lcu_context_kernels_per_step(self.handle)

    def set_sampling(self, mode, seed=0):
        check(lib.lcu_context_set_sampling(self.handle, mode, seed))

    def rollover(self, keep):
        check(lib.lcu_context_rollover(self.handle, keep))

    def bench_kernel(self, which, reps):
        ms, b = C.c_float(0), C.c_uint64(0)
        check(lib.lcu_bench_decode_kernel(self.handle, which, reps, C.byref(ms), C.byref(b)))
        return ms.value, b.value

    def close(self):
        if self.handle:
            lib.lcu_context_free(self.handle)
            self.handle = None


class TensorParallel:
    """Row-sharded model + context over several GPUs of one box (lcu_tp_*): the same calls as Context."""

    def __init__(self, n_gpus, dim, n_heads, n_layers, n_vocab, multiple_of=256, norm_eps=1e-6, block_size=0, context_len=2048,
                 temperature=0.9, gpus=None, seed=None, scale=0.02, path=None):
        self.n_vocab = n_vocab
        self.handle = vp()
        g = None if gpus is None else _ptr(np.ascontiguousarray(gpus, np.int32))
        check(lib.lcu_tp_create(pack_params(dim, multiple_of, n_heads, n_layers, n_vocab, norm_eps, block_size), g, n_gpus, context_len,
                                temperature, C.byref(self.handle)))
        if path is not None:
            check(lib.lcu_tp_load(self.handle, path.encode()))
        elif seed is not None:
            check(lib.lcu_tp_fill_synthetic(self.handle, seed, scale))

    def next_token(self, tokens):
        t = np.ascontiguousarray(np.asarray(tokens, np.int16))
        out = C.c_int(0)
        check(lib.lcu_tp_next_token(self.handle, _ptr(t), len(t), C.byref(out)))
        return out.value

    def decode_chained(self, first_token, n_steps):
        toks = np.empty(n_steps, np.int16)
        ms = C.c_float(0)
        check(lib.lcu_tp_decode_chained(self.handle, int(first_token), n_steps, _ptr(toks), C.byref(ms)))
        return toks, ms.value

    def probs(self):
        out = np.empty(self.n_vocab, np.uint16)
        check(lib.lcu_tp_read_probs(self.handle, _ptr(out)))
        return out

    def clear_tokens(self):
        lib.lcu_tp_clear_tokens(self.handle)

    def tokens_left(self):
        return lib.lcu_tp_tokens_left(self.handle)

    def kernels_per_step(self):
        return lib.lcu_tp_kernels_per_step(self.handle)

    def weight_bytes_per_gpu(self):
        return lib.lcu_tp_weight_bytes_per_gpu(self.handle)

    def close(self):
        if self.handle:
            lib.lcu_tp_free(self.handle)
            self.handle = None


def bench_matmul_f16_ms(m, k, n, reps=20, seed=7):
    """Mean milliseconds of one out(m,n) = lhs(m,k) . w(n,k)^T on seeded device-resident operands (CUDA events)."""
    x, w, o = DeviceBuffer(m * k * 2), DeviceBuffer(n * k * 2), DeviceBuffer(m * n * 2)
    check(lib.lcu_synth_fill_f16(x.ptr, m * k, seed, b"bench.x", 1.0, 0, None))
    check(lib.lcu_synth_fill_f16(w.ptr, n * k, seed, b"bench.w", 0.02, 0, None))
    ms = C.c_float(0)
    check(lib.lcu_bench_matmul_f16(o.ptr, x.ptr, w.ptr, m, k, n, reps, C.byref(ms)))
    return ms.value


def read_ceiling_ms(nbytes, reps=10, copies_per_stage=1):
    ms = C.c_float(0)
    check(lib.lcu_bench_read_ceiling(nbytes, reps, copies_per_stage, C.byref(ms)))
    return ms.value
