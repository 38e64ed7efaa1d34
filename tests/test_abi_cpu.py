"""The C-ABI library loads without a GPU, exports every declared symbol, and refuses to compute
without a device (no silent CPU path).  Host-side model/partition logic is checked as well."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import ROOT, load_package


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "llama_cu_c.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lcu_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lcu = load_package()
    names = declared_symbols()
    assert len(names) >= 45
    for n in names:
        assert hasattr(lcu.lib, n), f"{n} declared in include/llama_cu_c.h but not exported"
    assert set(lcu.EXPORTS) == set(names), set(lcu.EXPORTS) ^ set(names)


def test_no_cpu_fallback_without_a_device():
    lcu = load_package()
    if lcu.lib.lcu_device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(lcu.LcuError, match="no CUDA device"):
        lcu.quantize(np.zeros((2, 128), np.uint16), 128)
    with pytest.raises(lcu.LcuError, match="no CUDA device"):
        lcu.matmul_nt(np.zeros((1, 256), np.uint16), np.zeros((2, 256), np.uint16))
    with pytest.raises(lcu.LcuError, match="no CUDA device"):
        lcu.Model.synthetic(256, 2, 1, 1000)


def test_host_side_shapes_and_partitions():
    lcu = load_package()
    assert lcu.lib.lcu_ffn_dim(4096, 256) == 11008
    assert lcu.lib.lcu_ffn_dim(5120, 256) == 13824
    assert lcu.lib.lcu_ffn_dim(8192, 256) == 22016
    lg = np.zeros(80, np.int32)
    assert lcu.lib.lcu_partition_even(80, 8, lg.ctypes.data_as(C.c_void_p)) == 0
    assert (np.bincount(lg) == 10).all() and (np.diff(lg) >= 0).all()
    assert lcu.lib.lcu_partition_even(40, 2, lg.ctypes.data_as(C.c_void_p)) == 0
    assert lg[:40].tolist() == [0] * 20 + [1] * 20
    assert lcu.lib.lcu_partition_even(2, 4, lg.ctypes.data_as(C.c_void_p)) != 0
    assert b"partition" in lcu.lib.lcu_last_error()
    assert len(lcu.pack_params(4096, 256, 32, 32, 32000)) == 40
    assert lcu.lib.lcu_set_matmul_type(3) != 0 and lcu.lib.lcu_set_matmul_type(1) == 0 and lcu.lib.lcu_set_matmul_type(4) == 0


def test_short_prompt_gemm_plan_fills_one_wave():
    """Host arithmetic behind lcu_matmul_nt_f16 for up to 128 rows: the weights stream once and every SM takes in about the
    same rate, so the tile width and split-K factor are chosen for one wave of equal CTAs.  The plan for the reference's
    model shapes on a 148-SM GPU (7B: dim 4096 / ffn 11008, 13B: 5120 / 13824, 65B: 8192 / 22016)."""
    lcu = load_package()

    def plan(n, k, sms=148):
        tile, split = C.c_int(0), C.c_int(0)
        lcu.check(lcu.lib.lcu_plan_short_prompt_gemm(n, k, sms, C.byref(tile), C.byref(split)))
        return tile.value, split.value

    # 7B: w1|w3 stacked (N = 22016) as 138 tiles of 160 columns instead of 172 of 128 in two waves; wq|wk|wv as 128 x 96
    assert plan(22016, 4096) == (160, 1)
    assert plan(12288, 4096) == (96, 1)
    # narrow matrices keep 128-wide tiles and split K over a cluster
    assert plan(4096, 4096) == (128, 4)
    assert plan(4096, 11008) == (128, 4)
    # 13B and 65B
    assert plan(27648, 5120) == (192, 1)
    assert plan(24576, 8192) == (192, 1)
    for n, k in ((22016, 4096), (12288, 4096), (4096, 4096), (27648, 5120), (24576, 8192), (32000, 4096), (15360, 5120)):
        tile, split = plan(n, k)
        assert tile % 32 == 0 and 96 <= tile <= 256 and split in (1, 2, 4) and (split == 1 or tile == 128)
        ctas = -(-n // tile) * split
        assert 74 < ctas <= 148, (n, k, tile, split, ctas)  # one wave, more than half of the SMs busy
    # a GPU with half the SMs gets wider tiles
    assert plan(12288, 4096, 74)[0] > plan(12288, 4096, 148)[0]
    with pytest.raises(lcu.LcuError):
        plan(100, 4096)


def test_long_prompt_gemm_plan_follows_the_measurements():
    """Host arithmetic behind lcu_matmul_nt_f16 for more than 128 rows: whole tiles per SM pair (0) or the kernel that
    deals the last wave's K steps evenly (256).  Pinned where the two were measured more than 5 % apart on a B200 (7B
    shapes, microseconds whole / balanced in the comments)."""
    lcu = load_package()

    def plan(m, n, k, sms=148):
        out = C.c_int(-1)
        lcu.check(lcu.lib.lcu_plan_long_prompt_gemm(m, n, k, sms, C.byref(out)))
        return out.value

    assert plan(512, 22016, 4096) == 256    # 83.1 / 78.5: 172 tiles for 74 pairs, the third wave is a third full
    assert plan(2048, 22016, 4096) == 256   # 278 / 259
    assert plan(512, 4096, 4096) == 0       # 28.9 / 33.4: every tile would be handed over
    assert plan(768, 4096, 4096) == 256     # 48.9 / 34.3
    assert plan(512, 4096, 11008) == 256    # 82.4 / 66.1
    assert plan(1024, 4096, 11008) == 0     # 72.3 / 83.3: 64 tiles, one wave
    for m in (129, 300, 777, 2048, 8192):
        for n, k in ((4096, 4096), (12288, 4096), (22016, 4096), (27648, 5120), (8192, 22016), (32000, 4096)):
            assert plan(m, n, k) in (0, 256, 512)
    with pytest.raises(lcu.LcuError):
        plan(128, 4096, 4096)


def test_balanced_gemm_schedule_covers_every_k_step_once():
    """The prompt GEMM that deals the last wave's K steps evenly over the SM pairs: its work list, walked on the host for
    every pair of a launch.  Every K step of every tile must be run by exactly one pair; a pair may start inside a tile
    (and hand partial sums over) once at most, with its first shared segment; the pair that ran a shared tile's first K
    step must find exactly the following pairs that ran the rest, in order."""
    lcu = load_package()
    cases = 0
    for pairs in (1, 2, 3, 7, 37, 66, 74):
        for k_steps in (1, 2, 3, 5, 8, 64, 80, 172, 344):
            for n_tiles in list(range(1, 160)) + [172, 344, 516, 688, 1376]:
                assert lcu.lib.lcu_selftest_balanced_schedule(n_tiles, k_steps, pairs) == 0, (n_tiles, k_steps, pairs)
                cases += 1
    assert cases > 10000
    assert lcu.lib.lcu_selftest_balanced_schedule(0, 64, 74) == -1


def test_oracle_is_not_linked_into_the_product():
    out = subprocess.run(["nm", "-D", "--defined-only", os.path.join(ROOT, "llama.cu_b200", "libllama_cu_b200.so")],
                         capture_output=True, text=True).stdout
    assert "orc_" not in out and "ref_" not in out
    for root, _, files in os.walk(os.path.join(ROOT, "llama.cu_b200")):
        for f in files:
            if f.endswith((".cu", ".cuh", ".py", ".h")):
                src = open(os.path.join(root, f)).read()
                assert "oracle" not in src.lower().replace("oracle/liboracle", "") or f == "__init__.py" and "oracle" not in src, f


def test_tensor_parallel_split_rules():
    """Row shards need whole heads per GPU and even row counts of the ffn and output matrices: the three model sizes of
    the configurations split over 2, 4 and 8 GPUs; uneven splits are refused on the host."""
    lcu = load_package()
    for dim, heads in ((4096, 32), (5120, 40), (8192, 64)):
        raw = lcu.pack_params(dim, 256, heads, 2, 32000)
        for n in (2, 4, 8):
            assert lcu.lib.lcu_tp_check_split(raw, n) == 0, (dim, n, lcu.lib.lcu_last_error())
        assert lcu.lib.lcu_tp_check_split(raw, 3) != 0
    assert lcu.lib.lcu_tp_check_split(lcu.pack_params(5120, 256, 40, 2, 32000), 16) != 0
    assert lcu.lib.lcu_tp_check_split(lcu.pack_params(512, 256, 4, 2, 2001), 2) != 0 and b"vocabulary" in lcu.lib.lcu_last_error()


def test_partition_must_be_contiguous():
    """A GPU may not reappear after another one was used: the head runs on the last layer's GPU and the residual row is
    handed from stage to stage, so [0, 1, 0] would run the head against another stage's buffers."""
    lcu = load_package()
    ok = lambda lg: lcu.lib.lcu_partition_is_contiguous(np.asarray(lg, np.int32).ctypes.data_as(C.c_void_p), len(lg))
    assert ok([0, 0, 0]) == 1 and ok([0, 0, 1, 1, 3]) == 1 and ok([2, 2, 0, 1]) == 1
    assert ok([0, 1, 0]) == 0 and ok([0, 0, 1, 1, 0, 0]) == 0 and ok([1, 0, 2, 0]) == 0


@pytest.mark.parametrize("name,dim,heads,layers,bs", [("7B", 4096, 32, 32, 0), ("7B-u8", 4096, 32, 32, 128), ("13B", 5120, 40, 40, 0),
                                                      ("65B-u8", 8192, 64, 80, 128)])
def test_context_scratch_figure_counts_every_buffer(name, dim, heads, layers, bs):
    """One function sizes the per-GPU scratch arena for the context, the memory-based partitioner and
    llama_params::shared_context_memory_size.  It must cover the activations and, for u8 models, the dequantization
    buffers; the score buffer (heads x ctx x round_up(ctx, 128) halves) is part of it only while the three-kernel prompt
    attention is selected - the default one-kernel path keeps scores in tensor memory."""
    lcu = load_package()
    ctx = 2048
    ffn = lcu.lib.lcu_ffn_dim(dim, 256)
    raw = lcu.pack_params(dim, 256, heads, layers, 32000, 1e-6, bs)
    got = lcu.lib.lcu_context_scratch_bytes(raw, ctx)
    activations = 6 * ctx * dim * 2 + 3 * ctx * ffn * 2
    scores = 0
    lcu.check(lcu.lib.lcu_set_tuning(b"prefill_attn_tc", 1))
    try:
        with_scores = lcu.lib.lcu_context_scratch_bytes(raw, ctx)
    finally:
        lcu.check(lcu.lib.lcu_set_tuning(b"prefill_attn_tc", 2))
    assert with_scores - got >= heads * ctx * ((ctx + 127) // 128 * 128) * 2
    deq = 2 * max(2 * ffn * dim, 3 * dim * dim) * 2 if bs else 0  # two buffers: one feeds the GEMM in flight, the next matrix expands into the other
    tables = ctx * (dim // heads // 2) * 8 + 2 * 32000 * 2 + 2 * ctx * 2
    assert activations + scores + deq + tables <= got <= activations + scores + deq + tables + 64 * 256, name
    assert lcu.lib.lcu_context_kv_bytes_per_layer(raw, ctx) == 2 * ctx * dim * 2


REF = os.environ.get("REF", os.environ.get("LLAMA_CU_REFERENCE", "/root/reference"))


def linked_source(tmp_path, name):
    """A quoted #include is searched in the including file's directory first; reaching the reference's source through a
    symbolic link keeps its "llama_cu.h" from resolving to the reference's own header (nothing is copied)."""
    link = tmp_path / name
    os.symlink(os.path.join(REF, name), link)
    return str(link)


def header_used(compiler, src, *flags):
    deps = subprocess.run([compiler, "-std=c++17", "-I", os.path.join(ROOT, "include"), *flags, "-M", src], capture_output=True, text=True).stdout
    return [os.path.realpath(p) for p in re.findall(r"(\S*llama_cu\.h)", deps)]


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "transform.cu")), reason="reference sources not present")
def test_reference_transform_tool_builds_against_the_new_header_and_library(tmp_path):
    """The reference's transform.cu uses the LLAMA_CU_IMPLEMENTATION half of its header (tensor4d, gpu_buffer, generic_tensor,
    CHECK_CUDA, RETURN_UNLESS): unmodified, it must compile against include/llama_cu.h and link with the new library."""
    src = linked_source(tmp_path, "transform.cu")
    assert header_used("nvcc", src) == [os.path.join(ROOT, "include", "llama_cu.h")]
    exe = tmp_path / "transform"
    r = subprocess.run(["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "include"),
                        src, "-o", str(exe), "-L", os.path.join(ROOT, "llama.cu_b200"), "-lllama_cu_b200"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "main.cpp")), reason="reference sources not present")
def test_reference_main_compiles_against_the_new_header(tmp_path):
    """Drop-in proof at the source level: the reference's own client builds against include/llama_cu.h."""
    src = linked_source(tmp_path, "main.cpp")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    assert header_used(cxx, src) == [os.path.join(ROOT, "include", "llama_cu.h")]
    exe = tmp_path / "llama_cu_main"
    r = subprocess.run([cxx, "-std=c++17", "-I", os.path.join(ROOT, "include"), src, "-o", str(exe),
                        "-L", os.path.join(ROOT, "llama.cu_b200"), "-lllama_cu_b200",
                        "-Wl,-rpath," + os.path.join(ROOT, "llama.cu_b200")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
